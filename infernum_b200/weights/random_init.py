"""Random weights: either tensors on a device, or a whole model folder
(config.json + model.safetensors) written from a configuration and a seed.

Linear and embedding weights are N(0, std) with the std the part declares
(0.02), norm weights 1 + U(-0.1, 0.1).  A value is a function of (seed,
position of the tensor in the model's declaration, position of the element in
the tensor) alone, computed the same way on every device: the tensors drawn on
the GPU and the ones written to a folder for the same configuration and seed
are equal bit for bit, and a tensor does not depend on which others were drawn.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping, Optional

import torch

from ..parts.base import Runtime, WeightSpec
from .safetensors_io import write_safetensors


_M32 = 0xFFFFFFFF
_CHUNK = 1 << 25  # elements drawn at a time (bounds the temporaries for the largest tensors)
_TABLE_BITS = 16
_normal_tables: Dict[str, torch.Tensor] = {}


def _hash32(index: torch.Tensor, key: int) -> torch.Tensor:
    """A 32-bit mix of (element index, key), held in int64 and computed with
    integer operations only (multipliers below 2^31, so no product leaves 63
    bits): the same bits on every device."""
    x = (index ^ (key & _M32)) & _M32
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & _M32
    x = x ^ (x >> 15)
    x = (x * 0x2C1B3C6D) & _M32
    x = x ^ (x >> 16)
    x = (x + ((key >> 32) & _M32)) & _M32
    x = (x * 0x3243F6A9) & _M32
    x = x ^ (x >> 15)
    x = (x * 0x7FEB352D) & _M32
    return x ^ (x >> 16)


def _normal_table(device) -> torch.Tensor:
    """Quantiles of N(0, 1) at (i + 0.5) / 2^16, worked out once on the CPU in
    float64 and copied: every device interpolates in the same numbers."""
    key = str(device)
    t = _normal_tables.get(key)
    if t is None:
        base = _normal_tables.get("cpu")
        if base is None:
            n = 1 << _TABLE_BITS
            p = (torch.arange(n + 1, dtype=torch.float64) + 0.5) / (n + 1)
            base = torch.erfinv(2.0 * p - 1.0) * (2.0 ** 0.5)
            _normal_tables["cpu"] = base
        t = base.to(device)
        _normal_tables[key] = t
    return t


def _draw(spec: WeightSpec, key: int, device) -> torch.Tensor:
    """One tensor in float32.  Random values are a function of (key, element
    index) made of integer operations, one table look-up and exact float64
    arithmetic, so a tensor drawn on the GPU equals the one drawn on the CPU
    bit for bit: a model benchmarked from ``random_model`` can be written out
    with ``write_random_model`` and handed to another implementation."""
    shape = tuple(spec.shape)
    if spec.kind == "int":
        return torch.zeros(shape, dtype=torch.int32, device=device)
    if spec.init == "zeros":
        return torch.zeros(shape, dtype=torch.float32, device=device)
    if spec.init == "ones":
        return torch.ones(shape, dtype=torch.float32, device=device)
    if spec.init not in ("normal", "norm"):
        raise ValueError(f"unknown init {spec.init!r}")
    n = 1
    for d in shape:
        n *= int(d)
    out = torch.empty(n, dtype=torch.float32, device=device)
    table = _normal_table(device) if spec.init == "normal" else None
    for lo in range(0, n, _CHUNK):
        hi = min(n, lo + _CHUNK)
        h = _hash32(torch.arange(lo, hi, dtype=torch.int64, device=device), key)
        if spec.init == "normal":
            # the high bits pick a quantile, the low ones a place between it and the next
            i = h >> (32 - _TABLE_BITS)
            frac = (h & ((1 << (32 - _TABLE_BITS)) - 1)).to(torch.float64) / float(1 << (32 - _TABLE_BITS))
            a, b = table[i], table[i + 1]
            z = a + (b - a) * frac
            out[lo:hi] = (z * spec.std).to(torch.float32)
        else:
            u = h.to(torch.float64) / float(1 << 32)
            out[lo:hi] = (1.0 + (u - 0.5) * 0.2).to(torch.float32)
    return out.view(shape)


def _tensor_key(seed: int, index: int) -> int:
    return (int(seed) * 1_000_003 + index * 0x9E3779B97F4A7C15 + 0x1234567) & 0xFFFFFFFFFFFFFFFF


def random_tensors(specs: Mapping[str, WeightSpec], seed: int, device,
                   dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    """All tensors of a model drawn on ``device``, rounded to ``dtype``
    (through bfloat16 first, so that a float32 engine sees the same values a
    bfloat16 checkpoint would hold)."""
    device = torch.device(device)
    out = {}
    for idx, (name, spec) in enumerate(specs.items()):
        t = _draw(spec, _tensor_key(seed, idx), device)
        if spec.kind != "int":
            t = t.to(torch.bfloat16).to(dtype)
        out[name] = t
    return out


def model_specs_for(config: Mapping[str, Any]):
    """(typed config, ModelSpec, weight specs) of a config.json dict."""
    from ..models.model import Model
    from ..registry import resolve_config

    arch, cfg = resolve_config(config)
    spec = arch.build_spec(cfg)
    model = Model(spec, Runtime(device=torch.device("cpu"), dtype=torch.bfloat16))
    return cfg, spec, model.weight_specs()


def write_random_model(folder: str, config: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16, device: Optional[str] = None) -> str:
    """Writes ``folder/config.json`` and ``folder/model.safetensors``.  The
    tensors are drawn on ``device`` (default: a GPU if there is one, which is a
    hundred times faster for a large model) and are the same wherever they are drawn."""
    os.makedirs(folder, exist_ok=True)
    cfg, _, specs = model_specs_for(config)
    names = list(specs)
    index = {n: i for i, n in enumerate(names)}
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"

    def produce(name: str) -> torch.Tensor:
        spec = specs[name]
        t = _draw(spec, _tensor_key(seed, index[name]), device)
        return (t if spec.kind == "int" else t.to(dtype)).cpu()

    file_specs = [(n, torch.int32 if specs[n].kind == "int" else dtype, specs[n].shape)
                  for n in names]
    write_safetensors(os.path.join(folder, "model.safetensors"), file_specs, produce,
                      metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(dict(config), fh, indent=1)
    return folder
