"""Rotary position embedding, half-rotation pairing.

For pair index j in [0, rd/2) the elements (j, j + rd/2) of a head are rotated
by the angle ``p * f_j`` where p is the token's absolute position:
``y[j] = x[j] cos - x[j+rd/2] sin``, ``y[j+rd/2] = x[j] sin + x[j+rd/2] cos``
(infernum-cuda/kernels/rope.cu:25-41), ``f_j = theta^(-2j/rd)``
(infernum/src/rope.rs:24-27).  The angle is formed in 32-bit on the device from
the integer position and a float32 ``f_j``; there is no table and so no limit
from ``max_position_embeddings``.

``scaling`` of type "llama3" rescales the frequencies in three bands by
wavelength ``L_j = 2 pi / f_j`` against the original context length P:
L_j < P/high keeps f_j; L_j > P/low gives f_j / factor; between, with
``m = (P / L_j - low) / (high - low)``, ``f'_j = (1 - m) f_j / factor + m f_j``.
The reference has this ramp only in its YaRN branch with fixed bounds and an
extra magnitude factor (infernum/src/rope.rs:91-120); llama3 has no magnitude
factor.

Parameters: ``head_dim``, ``rotary_dim`` (default: head_dim), ``theta``,
``scaling`` (None or a dict with rope_type, factor, low_freq_factor,
high_freq_factor, original_max_position_embeddings).
"""

from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from ..errors import ConfigError
from ..ops import core
from .base import POSITION_ENCODINGS, PositionEncoding, Runtime


def rotary_inv_freq(rotary_dim: int, theta: float, scaling: Optional[Dict[str, Any]]) -> List[float]:
    """The rd/2 frequencies, computed in double precision on the host."""
    freqs = [theta ** (-2.0 * j / rotary_dim) for j in range(rotary_dim // 2)]
    if not scaling:
        return freqs
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return freqs
    if kind != "llama3":
        raise ConfigError(f"rotary scaling {kind!r} is not supported (supported: llama3)")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = []
    for f in freqs:
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / high:
            out.append(f)
        elif wavelen > orig / low:
            out.append(f / factor)
        else:
            m = (orig / wavelen - low) / (high - low)
            out.append((1.0 - m) * f / factor + m * f)
    return out


@POSITION_ENCODINGS.register("rotary")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ConfigError(f"rotary_dim {self.rotary_dim} must be even and within head_dim")
        self.theta = float(params["theta"])
        self.scaling = params.get("scaling")
        freqs = rotary_inv_freq(self.rotary_dim, self.theta, self.scaling)
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(rt.device)

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor) -> None:
        """Rotate q [N, heads, hd] and k [N, kv_heads, hd] in place."""
        for x in (q, k):
            if x is None:
                continue
            n, heads, hd = x.shape
            if x.stride(2) != 1 or x.stride(1) != hd:
                raise ConfigError("rotary apply: heads must be packed along each row")
            flat = x.as_strided((n, heads * hd), (x.stride(0), 1))
            core.rope_append(flat, positions, self.inv_freq, self.rotary_dim, heads, 0, hd,
                             None, None, None, None, self.rt.err)
