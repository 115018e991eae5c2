"""Random weights: either tensors on a device, or a whole model folder
(config.json + model.safetensors) written from a configuration and a seed.

Linear and embedding weights are N(0, std) with the std the part declares
(0.02), norm weights 1 + U(-0.1, 0.1).  Each tensor has its own generator
seeded from (seed, position of the tensor in the model's declaration), so a
tensor's values do not depend on which other tensors were drawn.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping

import torch

from ..parts.base import Runtime, WeightSpec
from .safetensors_io import write_safetensors


def _draw(spec: WeightSpec, gen: torch.Generator, device) -> torch.Tensor:
    shape = tuple(spec.shape)
    if spec.kind == "int":
        return torch.zeros(shape, dtype=torch.int32, device=device)
    if spec.init == "normal":
        return torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * spec.std
    if spec.init == "norm":
        return 1.0 + (torch.rand(shape, generator=gen, device=device, dtype=torch.float32) - 0.5) * 0.2
    if spec.init == "zeros":
        return torch.zeros(shape, dtype=torch.float32, device=device)
    if spec.init == "ones":
        return torch.ones(shape, dtype=torch.float32, device=device)
    raise ValueError(f"unknown init {spec.init!r}")


def random_tensors(specs: Mapping[str, WeightSpec], seed: int, device,
                   dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    """All tensors of a model drawn on ``device``, rounded to ``dtype``
    (through bfloat16 first, so that a float32 engine sees the same values a
    bfloat16 checkpoint would hold)."""
    device = torch.device(device)
    out = {}
    for idx, (name, spec) in enumerate(specs.items()):
        gen = torch.Generator(device=device)
        gen.manual_seed((int(seed) * 1_000_003 + idx) & 0x7FFFFFFFFFFFFFFF)
        t = _draw(spec, gen, device)
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
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes ``folder/config.json`` and ``folder/model.safetensors``."""
    os.makedirs(folder, exist_ok=True)
    cfg, _, specs = model_specs_for(config)
    names = list(specs)
    index = {n: i for i, n in enumerate(names)}

    def produce(name: str) -> torch.Tensor:
        spec = specs[name]
        gen = torch.Generator(device="cpu")
        gen.manual_seed((int(seed) * 1_000_003 + index[name]) & 0x7FFFFFFFFFFFFFFF)
        t = _draw(spec, gen, "cpu")
        return t if spec.kind == "int" else t.to(dtype)

    file_specs = [(n, torch.int32 if specs[n].kind == "int" else dtype, specs[n].shape)
                  for n in names]
    write_safetensors(os.path.join(folder, "model.safetensors"), file_specs, produce,
                      metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(dict(config), fh, indent=1)
    return folder
