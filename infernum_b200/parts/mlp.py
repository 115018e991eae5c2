"""SwiGLU feed-forward: ``d = (silu(x Wg^T) * (x Wu^T)) Wd^T`` with
``silu(g) = g / (1 + exp(-g))`` evaluated in 32-bit
(infernum-llama/src/graph_builder.rs:498-501; infernum-cuda/kernels/silu.cu:105-116).
Gate and up are one product with the row-concatenated weight ``[Wg; Wu]``.

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
        self.gate_up = Linear(torch.cat([gate, up], dim=0))
        self.down = Linear(weights[self.prefix + "down_proj.weight"])

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes + self.down.nbytes

    def forward(self, x: torch.Tensor, ctx=None) -> torch.Tensor:
        gu = self.gate_up(x)
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=gu.dtype, device=gu.device)
        core.silu_mul(gu, act)
        return self.down(act)
