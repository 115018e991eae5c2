"""From a model folder (or a configuration and a seed) to a model on the GPU."""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from .config.base import read_config_json
from .errors import ConfigError, KernelError
from .models.model import Model
from .parts.base import Runtime
from .registry import resolve_config
from .weights.loader import load_tensors
from .weights.random_init import random_tensors

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ConfigError(f"the engine runs in bfloat16 or float32, not {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ConfigError(f"unknown dtype {dtype!r}; use bfloat16 or float32") from None


def make_runtime(dtype, device="cuda:0", options: Optional[Dict[str, Any]] = None) -> Runtime:
    device = torch.device(device)
    if device.type != "cuda":
        raise KernelError(f"infernum_b200 runs on a CUDA device only, not on {device}")
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available; infernum_b200 has no CPU path")
    return Runtime(device=device, dtype=parse_dtype(dtype), options=dict(options or {}))


def load_model(folder: str, dtype="bfloat16", device="cuda:0",
               options: Optional[Dict[str, Any]] = None, strict: bool = True) -> Model:
    """Reads ``folder/config.json``, picks the architecture by its
    ``model_type``, and loads ``folder/*.safetensors`` by tensor name.
    ``strict=False`` turns tensors in the files that the model does not use from
    an error into a warning."""
    rt = make_runtime(dtype, device, options)
    arch, cfg = resolve_config(read_config_json(folder))
    spec = arch.build_spec(cfg)
    with torch.cuda.device(rt.device):
        model = Model(spec, rt)
        model.config = cfg
        weights = load_tensors(folder, model.weight_specs(), rt.dtype, rt.device, spec.ignorable, strict)
        model.bind(weights)
    return model


def random_model(config: Mapping[str, Any], seed: int = 0, dtype="bfloat16", device="cuda:0",
                 options: Optional[Dict[str, Any]] = None) -> Model:
    """A model with random weights drawn on the device (no files)."""
    rt = make_runtime(dtype, device, options)
    arch, cfg = resolve_config(config)
    spec = arch.build_spec(cfg)
    with torch.cuda.device(rt.device):
        model = Model(spec, rt)
        model.config = cfg
        model.bind(random_tensors(model.weight_specs(), seed, rt.device, rt.dtype))
    return model
