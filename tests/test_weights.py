"""Safetensors reading and writing, weight checks, random weights (no GPU)."""
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B
from infernum_b200.errors import WeightError
from infernum_b200.weights.loader import check_against_specs, kept_dtype
from infernum_b200.weights.random_init import model_specs_for, write_random_model
from infernum_b200.weights.safetensors_io import open_model_folder, save_tensors


def test_roundtrip_against_the_safetensors_library(tmp_path):
    from safetensors.torch import load_file, save_file

    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32),
               "c": torch.randn(2, 2, 2), "d": torch.zeros(0, 4)}
    ours = str(tmp_path / "ours.safetensors")
    save_tensors(ours, tensors)
    theirs = load_file(ours)
    for k, v in tensors.items():
        assert theirs[k].dtype == v.dtype and torch.equal(theirs[k], v)
    lib = str(tmp_path / "lib.safetensors")
    save_file(tensors, lib)
    table = open_model_folder(lib)
    for k, v in tensors.items():
        assert torch.equal(table[k].file.read(k), v)


def test_truncated_and_corrupt_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(WeightError, match="truncated"):
        open_model_folder(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightError, match="header length"):
        open_model_folder(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(WeightError, match="JSON"):
        open_model_folder(str(tmp_path))
    with pytest.raises(WeightError, match="no .safetensors"):
        open_model_folder(str(tmp_path / ".."/ "nothing-here") if False else str(_empty(tmp_path)))


def _empty(tmp_path):
    d = tmp_path / "empty"
    d.mkdir()
    return d


def test_random_model_folder_is_complete_and_seeded(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_A, seed=3)
    b = write_random_model(str(tmp_path / "b"), TINY_A, seed=3)
    c = write_random_model(str(tmp_path / "c"), TINY_A, seed=4)
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    ta, tb, tc = (open_model_folder(x) for x in (a, b, c))
    _, _, specs = model_specs_for(TINY_A)
    assert set(ta) == set(specs)
    assert "lm_head.weight" not in ta  # tied
    for name, e in ta.items():
        x = e.file.read(name)
        assert x.dtype == torch.bfloat16 and tuple(x.shape) == tuple(specs[name].shape)
        assert torch.equal(x, tb[name].file.read(name))
    assert not torch.equal(ta["model.norm.weight"].file.read("model.norm.weight"),
                           tc["model.norm.weight"].file.read("model.norm.weight"))
    w = ta["model.layers.0.mlp.up_proj.weight"].file.read("model.layers.0.mlp.up_proj.weight").float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = ta["model.norm.weight"].file.read("model.norm.weight").float()
    assert 0.89 <= n.min() and n.max() <= 1.11 and n.std() > 0.01  # bf16 rounds 1.1 up
    assert "lm_head.weight" in open_model_folder(write_random_model(str(tmp_path / "d"), TINY_B, 1))


def test_one_error_lists_everything(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_B, seed=1)
    table = dict(open_model_folder(folder))
    _, spec, specs = model_specs_for(TINY_B)
    check_against_specs(specs, table, spec.ignorable)  # fine as written

    from safetensors.torch import load_file, save_file
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    del tensors["model.layers.1.self_attn.k_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(5, 5, dtype=torch.bfloat16)
    tensors["stray.tensor"] = torch.zeros(3)
    tensors["model.layers.2.input_layernorm.weight"] = torch.zeros(96, dtype=torch.int32)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)  # ignorable
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.raises(WeightError) as exc:
        check_against_specs(specs, open_model_folder(folder), spec.ignorable)
    e = exc.value
    assert e.missing == ["model.layers.1.self_attn.k_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["stray.tensor"]
    assert e.wrong_shape == [("model.layers.0.mlp.down_proj.weight", (96, 256), (5, 5))]
    assert e.wrong_dtype == [("model.layers.2.input_layernorm.weight", "torch.int32")]
    text = str(e)
    for word in ("missing (2)", "unexpected (1)", "stray.tensor", "expected [96, 256]",
                 "file has [5, 5]", "k_proj"):
        assert word in text


def test_unused_tensors_can_be_a_warning_instead(tmp_path):
    """``strict=False``: a tensor nobody asked for is named in a warning (the
    reference ignores it); a missing one is an error either way."""
    folder = write_random_model(str(tmp_path / "m"), TINY_B, seed=1)
    _, spec, specs = model_specs_for(TINY_B)
    from safetensors.torch import load_file, save_file
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    tensors["stray.tensor"] = torch.zeros(3)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.raises(WeightError):
        check_against_specs(specs, open_model_folder(folder), spec.ignorable)
    with pytest.warns(UserWarning, match="stray.tensor"):
        src = check_against_specs(specs, open_model_folder(folder), spec.ignorable, strict=False)
    assert set(src) == set(specs)
    del tensors["model.norm.weight"]
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.warns(UserWarning), pytest.raises(WeightError) as exc:
        check_against_specs(specs, open_model_folder(folder), spec.ignorable, strict=False)
    assert exc.value.missing == ["model.norm.weight"] and exc.value.unexpected == []


def test_head_falls_back_to_the_embedding(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_B, seed=1)
    from safetensors.torch import load_file, save_file
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    del tensors["lm_head.weight"]
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    _, spec, specs = model_specs_for(TINY_B)
    src = check_against_specs(specs, open_model_folder(folder), spec.ignorable)
    assert src["lm_head.weight"] == "model.embed_tokens.weight"


def test_tied_model_ignores_a_stored_head(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, seed=1)
    from safetensors.torch import load_file, save_file
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    _, spec, specs = model_specs_for(TINY_A)
    check_against_specs(specs, open_model_folder(folder), spec.ignorable)


def test_kept_dtypes():
    from infernum_b200.parts.base import WeightSpec
    f, i = WeightSpec((1,)), WeightSpec((1,), kind="int")
    assert kept_dtype(f, torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert kept_dtype(f, torch.float16, torch.bfloat16) == torch.bfloat16
    assert kept_dtype(f, torch.float32, torch.bfloat16) == torch.float32  # stored 32-bit stays so
    assert kept_dtype(f, torch.bfloat16, torch.float32) == torch.float32
    assert kept_dtype(i, torch.int64, torch.bfloat16) == torch.int32
