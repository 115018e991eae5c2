"""Block arrangements.

``prenorm``: the Llama layer (infernum-llama/src/graph_builder.rs:451-507):
``h += mixer(norm1(h))``; ``h += ffn(norm2(h))``.  The two adds are not done
here: each output is pushed on the residual stream as a pending delta and the
next norm kernel folds it in (the reference's optimizer fuses add + rms_norm
the same way, infernum/src/graph/optimizer.rs:105-174).

Parts of a ``prenorm`` layer: ``norm1``, ``mixer``, ``norm2``, ``ffn``.
"""

from __future__ import annotations

from ..errors import ConfigError
from .base import BLOCKS, Block, ResidualStream


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, params, rt, parts):
        super().__init__(params, rt, parts)
        missing = [r for r in ("norm1", "mixer", "norm2", "ffn") if r not in parts]
        if missing:
            raise ConfigError(f"prenorm block {params.get('name', '')!r} lacks parts {missing}")

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        p = self.parts
        stream.push(p["mixer"].forward(p["norm1"].forward(stream), ctx, cache))
        stream.push(p["ffn"].forward(p["norm2"].forward(stream), ctx))
