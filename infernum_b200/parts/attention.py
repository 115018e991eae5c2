"""Grouped-query causal attention over the paged cache.

Per layer (infernum-llama/src/graph_builder.rs:456-483 for prefill, :819-864
for paged decode): q, k, v projections without bias; q -> [N, heads, hd],
k, v -> [N, kv_heads, hd]; position encoding on q and k; the new k and v are
written to the request's pages at the token's absolute position; query head a
reads kv head a / (heads / kv_heads); scores scaled by 1/sqrt(hd); causal
softmax in 32-bit; output projection.

The three projections are one product with the row-concatenated weight
``[Wq; Wk; Wv]`` (the reference does this for decode,
infernum-llama/src/graph_builder.rs:819-827); only the fused copy is kept.

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
``position`` (a position-encoding spec: {"kind", "params"}, or None),
``window`` (0 = all keys), ``scale`` (default 1/sqrt(head_dim)),
``prefix`` (checkpoint prefix, e.g. "model.layers.0.self_attn."),
``kv_shared`` (True: the layer has no k/v projection and reads the cache of
another run named by the schedule).
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..errors import ConfigError
from ..ops import attention as attn_ops
from ..ops import core
from .base import MIXERS, POSITION_ENCODINGS, Mixer, PagedCacheSpec, Runtime, WeightSpec
from .linear import Linear
from .rope import RotaryEmbedding


@MIXERS.register("attention")
class Attention(Mixer):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params.get("num_kv_heads", self.num_heads))
        self.head_dim = int(params["head_dim"])
        self.window = int(params.get("window") or 0)
        self.scale = float(params.get("scale") or 1.0 / math.sqrt(self.head_dim))
        self.prefix = params.get("prefix", "")
        self.kv_shared = bool(params.get("kv_shared", False))
        if self.num_heads % self.num_kv_heads:
            raise ConfigError(
                f"attention: {self.num_heads} heads are not a multiple of "
                f"{self.num_kv_heads} key/value heads")
        pos = params.get("position")
        self.position = None
        if pos:
            self.position = POSITION_ENCODINGS.get(pos["kind"])(pos.get("params", {}), rt)
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None

    # ---- declarations -----------------------------------------------------
    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return PagedCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        qd, kvd = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = {
            self.prefix + "q_proj.weight": WeightSpec((qd, self.hidden_size)),
            self.prefix + "o_proj.weight": WeightSpec((self.hidden_size, qd)),
        }
        if not self.kv_shared:
            specs[self.prefix + "k_proj.weight"] = WeightSpec((kvd, self.hidden_size))
            specs[self.prefix + "v_proj.weight"] = WeightSpec((kvd, self.hidden_size))
        return specs

    def bind(self, weights) -> None:
        names = ["q_proj.weight"] + ([] if self.kv_shared else ["k_proj.weight", "v_proj.weight"])
        mats = [weights[self.prefix + n] for n in names]
        if len({m.dtype for m in mats}) != 1:
            raise ConfigError(f"{self.prefix}: q/k/v projections are stored in different dtypes")
        self.qkv = Linear(torch.cat(mats, dim=0) if len(mats) > 1 else mats[0], self.rt)
        self.o = Linear(weights[self.prefix + "o_proj.weight"], self.rt)

    def weight_bytes(self) -> int:
        return self.qkv.nbytes + self.o.nbytes

    # ---- the step -----------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = self.qkv(x)  # [N, (nh + 2 nkv) hd], or [N, nh hd] when the cache is shared
        tables = ctx.block_tables[cache.group]
        writes = cache.owner and not self.kv_shared
        if self.kv_shared and cache.owner:
            raise ConfigError("a kv_shared attention layer must be scheduled with cache_of")
        rotary = self.position if isinstance(self.position, RotaryEmbedding) else None
        if self.position is not None and rotary is None:
            n = qkv.shape[0]
            q3 = qkv[:, : nh * hd].unflatten(1, (nh, hd))
            k3 = qkv[:, nh * hd: (nh + nkv) * hd].unflatten(1, (nkv, hd)) if writes else None
            self.position.apply(q3, k3, ctx.positions)
        core.rope_append(
            qkv, ctx.positions,
            rotary.inv_freq if rotary else None, rotary.rotary_dim if rotary else 0,
            nh, nkv if writes else 0, hd,
            ctx.row_entry if writes else None, tables if writes else None,
            cache.k_pool if writes else None, cache.v_pool if writes else None, self.rt.err)
        out = torch.empty((qkv.shape[0], nh * hd), dtype=qkv.dtype, device=qkv.device)
        attn_ops.paged_attention(qkv, cache.k_pool, cache.v_pool, out, ctx, tables, nh,
                                 self.scale, self.window, self.rt)
        return self.o(out)
