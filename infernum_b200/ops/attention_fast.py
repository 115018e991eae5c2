"""Tensor-core attention kernels for bfloat16 (``attention_mma.cu``), one
compiled module per head size, built when a model first needs it.

``run`` picks how the step's entries are spread: entries whose query rows
times grouped heads fit 8 packed rows (decoded tokens, very short portions)
go to split mode, where the keys of a request are cut in slices over several
CTAs and merged through scratch memory; longer portions go to tile mode.  It
returns False when there is no variant for the head size, and the caller then
takes the plain kernel.
"""

from __future__ import annotations

import ctypes
from typing import Dict

import torch

from ..csrc.build import load_module
from ..errors import KernelError
from . import core

_c_int, _c_float, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong
_libs: Dict[int, ctypes.CDLL] = {}
_tc_libs: Dict[int, ctypes.CDLL] = {}
SM_COUNT_FALLBACK = 148


def supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def lib_for(head_dim: int) -> ctypes.CDLL:
    lib = _libs.get(head_dim)
    if lib is None:
        lib = load_module(f"attn_hd{head_dim}", ["attention_mma.cu"], [f"-DIB_HD={head_dim}"])
        lib.ib_attention_mma.argtypes = [
            _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p,
            _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
            _c_float, _c_int, _c_int, _c_void_p, _c_ll, _c_void_p, _c_void_p]
        lib.ib_attention_mma.restype = _c_int
        lib.ib_attention_mma_scratch_bytes.argtypes = [_c_int, _c_int, _c_int]
        lib.ib_attention_mma_scratch_bytes.restype = _c_ll
        lib.ib_attention_mma_head_dim.restype = _c_int
        if lib.ib_attention_mma_head_dim() != head_dim:
            raise KernelError(f"attention module for head size {head_dim} was built for another size")
        _libs[head_dim] = lib
    return lib


def tc_lib_for(head_dim: int) -> ctypes.CDLL:
    """The tcgen05 prompt-attention module for a head size (64 or 128)."""
    lib = _tc_libs.get(head_dim)
    if lib is None:
        lib = load_module(f"attn_tc_hd{head_dim}", ["attention_tcgen05.cu"], [f"-DIB_HD={head_dim}"])
        lib.ib_attention_tc.argtypes = [
            _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
            _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int,
            _c_void_p, _c_void_p]
        lib.ib_attention_tc.restype = _c_int
        _tc_libs[head_dim] = lib
    return lib


def tc_eligible(q, k_pool, out, n_heads: int, window: int) -> bool:
    """Whether the tcgen05 prompt kernel takes this layer: head size 64 or 128,
    the head group a divisor of 128, pages of 8, 16, 32 or 64 tokens, no window,
    16-byte aligned rows."""
    _, nkv, page_size, hd = k_pool.shape
    G = n_heads // nkv
    return (hd in (64, 128) and window <= 0 and 128 % G == 0 and page_size % 8 == 0
            and 64 % page_size == 0 and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def choose_splits(n_entries: int, kv_heads_x_sub: int, max_kv_len: int, sm_count: int) -> int:
    """Slices per request in split mode.  Two CTAs fit an SM.  A CTA costs some
    microseconds beside its key tiles (start, first fetch, merging), during
    which its share of the SM streams nothing, so slices only pay while the
    unsliced grid leaves SMs idle (measured, 8 kv heads of 128, 148 SMs: 64
    requests of 1,100 keys take 51 us unsliced, 73 us in two slices; 8 requests
    19 us unsliced, 11 us in four slices; one request of 8,192 keys 99 us
    unsliced, 18 us in 8 slices, 15 us in 16).  Up to 8 slices are the CTAs of one
    cluster; more are merged by a second kernel, which pays only for very long
    single requests."""
    base = max(1, n_entries * kv_heads_x_sub)
    slots = 2 * sm_count
    tiles = max(1, -(-max_kv_len // 64))
    if 2 * base > slots:
        return 1
    if 16 * base <= slots and tiles >= 128:
        # (one request of 32,768 keys: 33 us in 16 slices, 30 us in 24, 31 us in 32)
        return 24 if tiles >= 256 and 10 * base * 24 <= 7 * slots else 16
    return max(1, min(8, slots // base, tiles))


def choose_prompt_splits(rows, rows_per_cta: int, nkv: int, max_kv_len: int, rt, small_limit: int = 0) -> int:
    """Into how many slices (1, 2 or 4 CTAs of one cluster) the prompt kernel
    cuts the keys of a row tile.  A portion of a few hundred tokens after a
    long cached prefix has few row tiles, each of which walks all the keys: 128
    CTAs for 512 tokens of 32 heads take 82 us over 4,096 keys, as long as
    1,024 tokens take.  Slices pay while the row tiles leave half of the CTA
    slots (two per SM) idle and every slice keeps at least eight key tiles."""
    if rows is None:
        return 1
    sm = rt.options.get("sm_count") or SM_COUNT_FALLBACK
    # (entries of at most small_limit rows are decoded tokens: another kernel takes them)
    ctas = sum(-(-r // rows_per_cta) for r in rows if r > small_limit) * nkv
    tiles = -(-max_kv_len // 64)
    for s in (4, 2):
        if ctas * s <= 2 * sm and tiles >= 8 * s:
            return s
    return 1


def _step_plan(ctx, G: int, nkv: int, tc_ok: bool, rt) -> dict:
    """How the entries of this step are spread over the kernels.  It depends on
    the step and on the layer's head grouping only, so it is worked out once per
    step (kept in ``ctx.scratch``), not once per layer."""
    key = ("attention_plan", G, nkv, tc_ok, getattr(ctx, "prompt_splits", None), getattr(ctx, "attention_mode", None))
    plan = ctx.scratch.get(key)
    if plan is not None:
        return plan
    gs = min(G, 8)  # split mode packs rows x grouped heads on the 8-wide side of the MMA
    n_hsub = -(-G // gs)
    small_limit = 8 // gs  # rows an entry may have to go to split mode
    sm = rt.options.get("sm_count") or SM_COUNT_FALLBACK
    cu = ctx.host_cu_rows
    rows = [cu[i + 1] - cu[i] for i in range(ctx.n_entries)]
    forced = getattr(ctx, "attention_mode", None)
    if forced is not None:
        mode, splits = forced
    else:
        any_small = any(r <= small_limit for r in rows)
        any_big = any(r > small_limit for r in rows)
        mode = (1 if any_big else 0) | (2 if any_small else 0)
        splits = choose_splits(ctx.n_entries, nkv * n_hsub, ctx.max_kv_len, sm) if mode == 2 else 1
    plan = {"mode": mode, "splits": splits, "prompt_splits": 1, "first_prompt_entry": 0,
            "splits_beside_prompts": splits}
    if (mode & 1) and tc_ok:
        beside = bool(mode & 2)
        plan["prompt_splits"] = getattr(ctx, "prompt_splits", None) or choose_prompt_splits(
            rows, 128 // G, nkv, ctx.max_kv_len, rt, small_limit if beside else 0)
        # decoded tokens come first in a step: the prompt kernel's grid starts at the first longer entry
        plan["first_prompt_entry"] = next((i for i, r in enumerate(rows) if r > small_limit), 0) if beside else 0
        if beside and forced is None:
            # the decoded tokens beside prompts are sliced as in a step of their own: a single
            # CTA per request and kv head would walk a long context tile by tile
            n_small = sum(1 for r in rows if r <= small_limit)
            plan["splits_beside_prompts"] = min(8, choose_splits(n_small, nkv * n_hsub, ctx.max_kv_len, sm))
    ctx.scratch[key] = plan
    return plan


def run(q, k_pool, v_pool, out, ctx, tables, n_heads, scale, window, rt) -> bool:
    num_pages, nkv, page_size, hd = k_pool.shape
    if not supported(hd):
        return False
    core.require_cuda(q, k_pool, v_pool, out, tables)
    if n_heads % nkv:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {nkv} kv heads")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.dtype != torch.bfloat16 \
            or k_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_mma: bfloat16 tensors with unit inner stride are required")
    G = n_heads // nkv
    tc_ok = rt.options.get("prompt_attention", "tcgen05") == "tcgen05" and tc_eligible(q, k_pool, out, n_heads, window)
    plan = _step_plan(ctx, G, nkv, tc_ok, rt)
    mode, splits = plan["mode"], plan["splits"]
    if (mode & 1) and tc_ok:
        # prompt portions on the tcgen05 kernel; what is left (decoded tokens and
        # very short portions in the same step) goes to split mode below
        code = tc_lib_for(hd).ib_attention_tc(
            q.data_ptr(), q.stride(0), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
            out.stride(0), ctx.cu_rows.data_ptr(), ctx.q_start.data_ptr(), tables.data_ptr(),
            tables.shape[1], ctx.n_entries, ctx.n_rows, ctx.max_rows_per_entry, n_heads, nkv,
            page_size, num_pages, float(scale), 8 if (mode & 2) else -1, plan["prompt_splits"],
            plan["first_prompt_entry"], rt.err.data_ptr(), core.stream_ptr(q))
        core.check(code, "attention_tcgen05")
        if not (mode & 2):
            return True
        mode = 2 | 4  # split mode for the small entries only; the others are done
        splits = plan["splits_beside_prompts"]
    if rt.options.get("split_copy", "tma") != "tma":
        mode |= 8  # keys and values by cp.async also where TMA could fetch them
    lib = lib_for(hd)
    scratch_ptr, scratch_bytes = None, 0
    if splits > 8:
        need = lib.ib_attention_mma_scratch_bytes(ctx.n_rows, n_heads, splits)
        buf = ctx.scratch.get("attn_split")
        if buf is None or buf.numel() * 4 < need:
            buf = torch.empty((need + 3) // 4, dtype=torch.float32, device=q.device)
            ctx.scratch["attn_split"] = buf
        scratch_ptr, scratch_bytes = buf.data_ptr(), buf.numel() * 4
    code = lib.ib_attention_mma(
        q.data_ptr(), q.stride(0), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
        out.stride(0), ctx.cu_rows.data_ptr(), ctx.q_start.data_ptr(), tables.data_ptr(),
        tables.shape[1], ctx.n_entries, ctx.n_rows, ctx.max_rows_per_entry, n_heads, nkv,
        page_size, num_pages, int(window), float(scale), mode, splits,
        scratch_ptr, scratch_bytes, rt.err.data_ptr(), core.stream_ptr(q))
    core.check(code, "attention_mma")
    return True
