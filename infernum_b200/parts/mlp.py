"""SwiGLU feed-forward: ``d = (silu(x Wg^T) * (x Wu^T)) Wd^T`` with
``silu(g) = g / (1 + exp(-g))`` evaluated in 32-bit
(infernum-llama/src/graph_builder.rs:498-501; infernum-cuda/kernels/silu.cu:105-116).
Gate and up are one product.  When the intermediate size is a multiple of 64
the fused weight interleaves them 64 rows by 64 rows ([g0..g63, u0..u63,
g64..g127, u64..u127, ...]), so that one 128-row tile of the tcgen05 product
holds gates and their ups and SiLU(gate) * up can be applied in its epilogue;
otherwise it is the plain concatenation ``[Wg; Wu]``.  Only the fused copy is
kept.

Parameters: ``hidden_size``, ``intermediate_size``, ``prefix`` (checkpoint
prefix, e.g. "model.layers.0.mlp.").
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import ConfigError
from ..ops import core
from .base import FEED_FORWARDS, FeedForward, Runtime, WeightSpec
from .linear import Linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.prefix = params.get("prefix", "")
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {
            self.prefix + "gate_proj.weight": WeightSpec((i, h)),
            self.prefix + "up_proj.weight": WeightSpec((i, h)),
            self.prefix + "down_proj.weight": WeightSpec((h, i)),
        }

    def bind(self, weights) -> None:
        gate = weights[self.prefix + "gate_proj.weight"]
        up = weights[self.prefix + "up_proj.weight"]
        if gate.dtype != up.dtype:
            raise ConfigError(f"{self.prefix}: gate and up projections are stored in different dtypes")
        i, h = self.intermediate_size, self.hidden_size
        self.block = None  # None: [all gates | all ups]; 64: interleaved 64 by 64
        if i % 64 == 0:
            fused = torch.stack([gate.view(i // 64, 64, h), up.view(i // 64, 64, h)], dim=1)
            self.gate_up = Linear(fused.reshape(2 * i, h), self.rt)
            self.block = 64
        else:
            self.gate_up = Linear(torch.cat([gate, up], dim=0), self.rt)
        self.down = Linear(weights[self.prefix + "down_proj.weight"], self.rt)

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes + self.down.nbytes

    def forward(self, x: torch.Tensor, ctx=None) -> torch.Tensor:
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        fused = False
        if self.block == 64 and x.dtype == torch.bfloat16 and self.gate_up.weight.dtype == torch.bfloat16:
            from ..ops import gemm_tc

            fused = gemm_tc.swiglu_route(x, self.gate_up.weight, act, self.gate_up.err)
        if not fused:
            core.silu_mul(self.gate_up(x), act, block=self.block)
        return self.down(act)
