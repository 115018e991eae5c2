"""RMSNorm: ``y = x * rsqrt(mean(x^2) + eps) * w`` (the weight multiplies
directly, no ``1 + w``), sum of squares and rsqrt in 32-bit, one rounding at
the store.  Reference: infernum-cuda/kernels/rmsnorm.cu:64-94 and, fused with
the residual add, infernum-cuda/kernels/add_rmsnorm.cu:78-108.

Parameters: ``hidden_size``, ``eps``, ``weight`` (checkpoint tensor name).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import core
from .base import NORMS, Norm, ResidualStream, Runtime, WeightSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.weight_name = params["weight"]
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.hidden_size,), init="norm")}

    def bind(self, weights) -> None:
        self.weight = weights[self.weight_name].contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, stream: ResidualStream, row_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        residual = stream.residual
        n_out = residual.shape[0] if row_idx is None else row_idx.numel()
        out = torch.empty((n_out, self.hidden_size), dtype=self.rt.dtype, device=residual.device)
        core.add_rmsnorm(residual, stream.pending, self.weight, self.eps, out, row_idx=row_idx,
                         write_residual=row_idx is None)
        if row_idx is None:
            stream.pending = None
        return out

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        core.add_rmsnorm(x, None, self.weight, self.eps, out)
        return out
