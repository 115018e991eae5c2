"""Loads a model's tensors from safetensors by name.

The model declares what it wants (name -> shape, kind); the files are checked
against that declaration in one pass and every fault is reported together:
missing tensors, tensors nobody asked for, wrong shapes and unusable dtypes.
(The reference walks the model's list and stops at the first missing name,
and does not check shapes: infernum-cuda/src/inner/cuda_graph_engine.rs:212-264,
infernum/src/weights/safetensors.rs:123-131.)

Kept dtypes: floating tensors stay bfloat16; float16 is converted to
bfloat16; a tensor stored in float32 stays float32 (the kernels take either);
integer tensors become int32.  An engine that runs in float32 widens every
floating tensor to float32, which is exact.
"""

from __future__ import annotations

import fnmatch
from typing import Dict, Iterable, Mapping

import torch

from ..errors import WeightError
from ..parts.base import WeightSpec
from .safetensors_io import TensorEntry, open_model_folder

_FLOAT_FILE_DTYPES = (torch.bfloat16, torch.float16, torch.float32)
_INT_FILE_DTYPES = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def check_against_specs(specs: Mapping[str, WeightSpec], table: Mapping[str, TensorEntry],
                        ignorable: Iterable[str] = (), strict: bool = True) -> Dict[str, str]:
    """Returns name -> source name in the files; raises one WeightError that
    lists everything that is wrong.  ``strict=False``: tensors nobody asked
    for are named in a warning instead (the reference ignores them silently);
    missing tensors, wrong shapes and unusable dtypes are errors either way."""
    missing, wrong_shape, wrong_dtype = [], [], []
    source: Dict[str, str] = {}
    for name, spec in specs.items():
        src = name if name in table else (spec.fallback if spec.fallback in table else None)
        if src is None:
            missing.append(name)
            continue
        entry = table[src]
        if tuple(entry.shape) != tuple(spec.shape):
            wrong_shape.append((name, tuple(spec.shape), tuple(entry.shape)))
        allowed = _INT_FILE_DTYPES if spec.kind == "int" else _FLOAT_FILE_DTYPES
        if entry.dtype not in allowed:
            wrong_dtype.append((name, str(entry.dtype)))
        source[name] = src
    used = set(source.values())
    patterns = list(ignorable)
    unexpected = sorted(
        n for n in table
        if n not in used and n not in specs and not any(fnmatch.fnmatchcase(n, p) for p in patterns)
    )
    if unexpected and not strict:
        import warnings

        warnings.warn(f"checkpoint holds {len(unexpected)} tensor(s) the model does not use: "
                      + ", ".join(unexpected[:8]) + (" ..." if len(unexpected) > 8 else ""), stacklevel=3)
        unexpected = []
    if missing or unexpected or wrong_shape or wrong_dtype:
        lines = ["checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, want, got in wrong_shape:
            lines.append(f"  wrong shape: {name} expected {list(want)}, file has {list(got)}")
        for name, got in wrong_dtype:
            lines.append(f"  unusable dtype: {name} is stored as {got}")
        raise WeightError("\n".join(lines), missing=sorted(missing), unexpected=unexpected,
                          wrong_shape=wrong_shape, wrong_dtype=wrong_dtype)
    return source


def kept_dtype(spec: WeightSpec, file_dtype: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    if spec.kind == "int":
        return torch.int32
    if engine_dtype == torch.float32 or file_dtype == torch.float32:
        return torch.float32
    return torch.bfloat16


def load_tensors(folder: str, specs: Mapping[str, WeightSpec], engine_dtype: torch.dtype,
                 device, ignorable: Iterable[str] = (), strict: bool = True) -> Dict[str, torch.Tensor]:
    table = open_model_folder(folder)
    source = check_against_specs(specs, table, ignorable, strict)
    out: Dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        entry = table[source[name]]
        cpu = entry.file.read(entry.name)
        dtype = kept_dtype(spec, entry.dtype, engine_dtype)
        # copy first (the mapped memory is read-only), convert on the device
        out[name] = cpu.to(device=device, copy=True).to(dtype)
    return out
