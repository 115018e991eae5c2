"""Chooses the attention kernel for a step.

``float32`` engines always take the plain kernel (one warp per row and head,
32-bit throughout).  ``bfloat16`` engines take the tensor-core prefill kernel
and the split-KV decode kernel when the head size has a compiled variant, and
the plain kernel otherwise; ``rt.options["attention"] = "plain"`` forces the
plain kernel (tests use it to compare the two).
"""

from __future__ import annotations

import torch

from . import core


def paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    out: torch.Tensor, ctx, tables: torch.Tensor, n_heads: int, scale: float,
                    window: int, rt) -> None:
    """Attention of every row of the step over its request's pages.

    ``q`` holds the (already position-encoded) queries in its first
    ``n_heads * head_dim`` columns; keys and values of the step's own tokens
    are already in the pools."""
    impl = rt.options.get("attention", "auto")
    if q.dtype == torch.bfloat16 and impl != "plain":
        from . import attention_fast

        if attention_fast.run(q, k_pool, v_pool, out, ctx, tables, n_heads, scale, window, rt):
            return
    core.attention_plain(q, k_pool, v_pool, out, ctx.positions, ctx.row_entry, tables, n_heads,
                         scale, window, rt.err)
