"""Typed configuration of the Llama dense decoder (``model_type: "llama"``).

Fields and defaults follow the reference's ``LlamaConfig``
(infernum-llama/src/config.rs:19-102, defaults :104-126): ``vocab_size``,
``hidden_size``, ``intermediate_size``, ``num_hidden_layers`` and
``num_attention_heads`` are required; ``num_key_value_heads`` defaults to the
head count, ``max_position_embeddings`` to 2048, ``rms_norm_eps`` to 1e-5,
``rope_theta`` to 10000, ``tie_word_embeddings`` to false, ``bos_token_id`` to
1 and ``eos_token_id`` to 2 (first element when it is a list).

Two keys go beyond the reference, which derives the head size as
``hidden_size / num_attention_heads`` (config.rs:264-266) and reads no
``rope_scaling`` for this family: an explicit ``head_dim``, and
``rope_scaling`` of ``rope_type: "llama3"``.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from ..errors import ConfigError
from .base import read_config_json, take_bool, take_float, take_int, take_int_or_first


@dataclass(frozen=True)
class Llama3RopeScaling:
    """The three-band frequency scaling that ``rope_type: "llama3"`` names."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int
    rope_type: str = "llama3"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> Optional["Llama3RopeScaling"]:
        if not isinstance(d, Mapping):
            raise ConfigError("config.json: 'rope_scaling' must be an object")
        rope_type = d.get("rope_type", d.get("type"))
        if rope_type in (None, "default"):
            return None
        if rope_type != "llama3":
            raise ConfigError(
                f"config.json: rope_scaling.rope_type {rope_type!r} is not supported "
                "for model_type 'llama' (supported: 'llama3', 'default')"
            )
        scaling = cls(
            factor=take_float(d, "factor"),
            low_freq_factor=take_float(d, "low_freq_factor"),
            high_freq_factor=take_float(d, "high_freq_factor"),
            original_max_position_embeddings=take_int(d, "original_max_position_embeddings"),
        )
        if scaling.factor <= 0:
            raise ConfigError("config.json: rope_scaling.factor must be > 0")
        if scaling.high_freq_factor <= scaling.low_freq_factor:
            raise ConfigError(
                "config.json: rope_scaling.high_freq_factor must exceed low_freq_factor"
            )
        return scaling

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[Llama3RopeScaling] = None
    tie_word_embeddings: bool = False
    bos_token_id: int = 1
    eos_token_id: int = 2
    model_type: str = "llama"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        model_type = d.get("model_type", "llama")
        if model_type != "llama":
            raise ConfigError(f"LlamaConfig cannot read model_type {model_type!r}")
        heads = take_int(d, "num_attention_heads")
        hidden = take_int(d, "hidden_size")
        head_dim = take_int(d, "head_dim", default=None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not divisible by "
                    f"num_attention_heads {heads} and no 'head_dim' is given"
                )
            head_dim = hidden // heads
        kv_heads = take_int(d, "num_key_value_heads", default=heads)
        scaling = d.get("rope_scaling")
        for key in ("attention_bias", "mlp_bias"):
            if take_bool(d, key, False):
                raise ConfigError(
                    f"config.json: '{key}': true is not supported (this architecture has no bias)"
                )
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (only 'silu')")
        cfg = cls(
            vocab_size=take_int(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=take_int(d, "intermediate_size"),
            num_hidden_layers=take_int(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=take_int(d, "max_position_embeddings", default=2048),
            rms_norm_eps=take_float(d, "rms_norm_eps", default=1e-5),
            rope_theta=take_float(d, "rope_theta", default=10000.0),
            rope_scaling=None if scaling is None else Llama3RopeScaling.from_dict(scaling),
            tie_word_embeddings=take_bool(d, "tie_word_embeddings", False),
            bos_token_id=take_int_or_first(d, "bos_token_id", 1),
            eos_token_id=take_int_or_first(d, "eos_token_id", 2),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_file(cls, path: str) -> "LlamaConfig":
        return cls.from_dict(read_config_json(path))

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} must be a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}"
            )
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary embedding")
        if self.rms_norm_eps <= 0:
            raise ConfigError("rms_norm_eps must be > 0")
        if self.rope_theta <= 0:
            raise ConfigError("rope_theta must be > 0")

    def to_dict(self) -> dict:
        d = dataclasses.asdict(self)
        if self.rope_scaling is None:
            d.pop("rope_scaling")
        d["architectures"] = ["LlamaForCausalLM"]
        return d
