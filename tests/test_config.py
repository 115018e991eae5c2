"""Typed configuration and the architecture registry (no GPU)."""
import json

import pytest

from helpers import TINY_A, TINY_B
from infernum_b200.config.llama import LlamaConfig
from infernum_b200.errors import ConfigError, UnsupportedModelError
from infernum_b200.parts.rope import rotary_inv_freq
from infernum_b200.registry import (register_architecture, resolve, resolve_config,
                                    supported_architectures)

MINIMAL = {"vocab_size": 100, "hidden_size": 48, "intermediate_size": 96, "num_hidden_layers": 2,
           "num_attention_heads": 4}


def test_defaults_follow_the_reference():
    cfg = LlamaConfig.from_dict(MINIMAL)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 12
    assert cfg.max_position_embeddings == 2048 and cfg.rms_norm_eps == 1e-5
    assert cfg.rope_theta == 10000.0 and cfg.rope_scaling is None
    assert cfg.tie_word_embeddings is False and cfg.bos_token_id == 1 and cfg.eos_token_id == 2
    assert cfg.model_type == "llama"


def test_every_key_is_read():
    cfg = LlamaConfig.from_dict(TINY_B)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads) == (3, 96, 3)
    assert (cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size) == (1, 32, 256)
    assert cfg.vocab_size == 320 and cfg.rope_theta == 500000.0 and cfg.rms_norm_eps == 1e-6
    sc = cfg.rope_scaling
    assert (sc.factor, sc.low_freq_factor, sc.high_freq_factor) == (8.0, 1.0, 4.0)
    assert sc.original_max_position_embeddings == 64
    assert LlamaConfig.from_dict(cfg.to_dict()) == cfg


def test_eos_list_takes_first():
    cfg = LlamaConfig.from_dict({**MINIMAL, "eos_token_id": [7, 8, 9]})
    assert cfg.eos_token_id == 7
    with pytest.raises(ConfigError):
        LlamaConfig.from_dict({**MINIMAL, "eos_token_id": []})


@pytest.mark.parametrize("key", sorted(MINIMAL))
def test_missing_required_key_names_it(key):
    d = dict(MINIMAL)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(d)


@pytest.mark.parametrize("patch, word", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 7}, "even"),
    ({"hidden_size": 50}, "divisible"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "gelu"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_bad_values_are_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict({**MINIMAL, **patch})


def test_registry_resolves_by_model_type(tmp_path):
    assert "llama" in supported_architectures()
    arch, cfg = resolve_config(TINY_A)
    assert arch.name == "llama" and cfg.hidden_size == 64
    arch, cfg = resolve_config({k: v for k, v in TINY_A.items() if k != "model_type"})
    assert arch.name == "llama"  # a missing model_type means llama
    with pytest.raises(UnsupportedModelError, match="mamba.*llama"):
        resolve("mamba")


def test_registry_takes_new_architectures():
    register_architecture("toy-arch", lambda d: d, lambda cfg: None)
    assert resolve("toy-arch").name == "toy-arch"


def test_spec_carries_every_size():
    arch, cfg = resolve_config(TINY_B)
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 3 and [s.layer for s in spec.schedule] == [0, 1, 2]
    mixer = spec.layers[1].parts["mixer"].params
    assert (mixer["num_heads"], mixer["num_kv_heads"], mixer["head_dim"]) == (3, 1, 32)
    assert mixer["position"]["params"]["theta"] == 500000.0
    assert spec.layers[0].parts["norm1"].params["eps"] == 1e-6
    assert spec.layers[2].parts["ffn"].params["intermediate_size"] == 256
    assert "tied_to" not in spec.lm_head.params
    arch, cfg = resolve_config(TINY_A)
    assert arch.build_spec(cfg).lm_head.params["tied_to"] == "model.embed_tokens.weight"


def test_llama3_bands_of_tiny_b():
    # head_dim 32: pairs 0,1 keep their frequency, 2 is interpolated, the rest is divided by 8
    base = rotary_inv_freq(32, 500000.0, None)
    scaled = rotary_inv_freq(32, 500000.0, TINY_B["rope_scaling"])
    assert scaled[0] == base[0] and scaled[1] == base[1]
    assert base[2] / 8 < scaled[2] < base[2]
    for j in range(3, 16):
        assert scaled[j] == pytest.approx(base[j] / 8, rel=1e-12)
