"""Token embedding and output head.

Embedding: ``h[t, :] = E[id_t, :]`` with no scaling
(infernum-llama/src/graph_builder.rs:442; infernum-cuda/kernels/embed.cu:36-50),
written straight into the float32 residual stream.

Head: ``logits = f . W_out^T`` on the rows whose logits are wanted, returned in
float32 from the 32-bit accumulator (the reference rounds them to bf16 first,
infernum-cuda/src/inner/cuda_graph_engine.rs:1297,1368).  ``tied_to`` makes the
head use the embedding table; otherwise a missing head tensor falls back to it
as in the reference (cuda_graph_engine.rs:225-232).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import core
from .base import EMBEDDINGS, HEADS, Part, Runtime, WeightSpec
from .linear import Linear


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.weight_name = params["weight"]
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size))}

    def bind(self, weights) -> None:
        self.weight = weights[self.weight_name].contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.numel(), self.hidden_size), dtype=torch.float32,
                          device=token_ids.device)
        core.embed(token_ids, self.weight, out, self.rt.err)
        return out


@HEADS.register("linear_head")
class LinearHead(Part):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.weight_name = params["weight"]
        self.tied_to = params.get("tied_to")
        self.fallback = params.get("fallback")
        self.proj: Optional[Linear] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        if self.tied_to:
            return {}
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size),
                                             fallback=self.fallback)}

    def bind(self, weights) -> None:
        self.proj = Linear(weights[self.tied_to or self.weight_name], self.rt)

    def weight_bytes(self) -> int:
        return self.proj.nbytes

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(x, out_dtype=torch.float32)
