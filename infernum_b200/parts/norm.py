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
from .base import NORMS, DeferredProduct, Norm, ResidualStream, Runtime, WeightSpec


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

    can_leave_row_factor = True

    def forward(self, stream: ResidualStream, row_idx: Optional[torch.Tensor] = None, scaled_ok: bool = False):
        """The normed rows.  With ``scaled_ok``, where the pending delta is a
        product still to be computed and its kernel can do it: one kernel runs
        that product, adds it to the residual and writes the rows times this
        norm's weights, with their sums of squares beside them (``ScaledRows``);
        the product that takes those rows applies the row factor."""
        residual = stream.residual
        if scaled_ok and row_idx is None and isinstance(stream.pending, DeferredProduct):
            from ..ops import gemm_tc

            pend = stream.pending
            rows = gemm_tc.add_norm_route(pend.x, pend.linear.weight, residual, self.weight, self.eps, pend.linear.err)
            if rows is not None:
                stream.pending = None
                return rows
        pending = stream.take_pending()
        n_out = residual.shape[0] if row_idx is None else row_idx.numel()
        out = torch.empty((n_out, self.hidden_size), dtype=self.rt.dtype, device=residual.device)
        core.add_rmsnorm(residual, pending, self.weight, self.eps, out, row_idx=row_idx,
                         write_residual=row_idx is None)
        if row_idx is None:
            stream.pending = None
        return out

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        core.add_rmsnorm(x, None, self.weight, self.eps, out)
        return out
