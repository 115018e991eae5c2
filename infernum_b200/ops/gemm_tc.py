"""The package's own bf16 matrix product on tcgen05 tensor cores
(``gemm_tcgen05.cu``): ``out[T, N] = x[T, K] @ w[N, K]^T`` with float32
accumulation in tensor memory, operands fetched by TMA.

``route`` is registered with ``parts.linear`` and takes a product when the
operands meet TMA's rules (16-byte aligned bases, row strides a multiple of 8
elements) and the policy admits the token count; otherwise the caller falls
back to the library GEMM.  K is split over several CTAs when the output alone
would leave most SMs idle (decode); the slices are the CTAs of one cluster
and are added in a fixed order through distributed shared memory.
"""

from __future__ import annotations

import ctypes
import functools
import os
from typing import Dict, Optional, Tuple

import torch

from ..csrc.build import load_module
from . import core

_c_int, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong
_lib: Optional[ctypes.CDLL] = None
_pair_lib: Optional[ctypes.CDLL] = None
_workspaces: Dict[torch.device, dict] = {}

BM, BK = 128, 64
# What a tile of gemm_pair costs beside its width, in weight rows: its token half is
# fetched and its prologue and epilogue run whatever the width.
PAIR_TILE_OVERHEAD = 66

# Which products the kernel takes: "all", "none", or a largest token count.
POLICY = {"mode": os.environ.get("INFERNUM_GEMM", "auto"), "max_tokens": 64, "pair_max_padding": 1.13,
          "pair_min_tokens_plain": 600, "pair_group_bytes": 64 << 20, "pair_group_max_tiles": 16,
          "sm_count": 148}


def pair_suits(T: int, fused_activation: bool = False) -> bool:
    """The kernel on pairs of SMs works on 256 tokens at a time; it is taken when
    rounding ``T`` up to that wastes little (measured on the 8B gate/up product
    with its activation: ahead of the library product plus activation kernel at
    256, 512, 768, 1024 and 2048 tokens, behind them at 320 and 520).  A plain
    product has too few tiles for the 74 pairs below three token tiles (the O
    product at 256 tokens: 18 us against the library's 11; at 512: 18.6 against
    14.8; at 768: 21.2 against 21.1), so it is taken from ``pair_min_tokens_plain``
    tokens on."""
    if not fused_activation and T < POLICY["pair_min_tokens_plain"]:
        return False
    return -(-T // 256) * 256 <= POLICY["pair_max_padding"] * T


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        l = load_module("gemm_tc", ["gemm_tcgen05.cu"])
        l.ib_gemm_tc.argtypes = [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int,
                                 _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p]
        l.ib_gemm_tc.restype = _c_int
        l.ib_gemm_tc_token_tile.argtypes = [_c_int]
        l.ib_gemm_tc_token_tile.restype = _c_int
        if torch.cuda.is_available():
            POLICY["sm_count"] = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        _lib = l
    return _lib


def pair_lib() -> ctypes.CDLL:
    """The kernel for many tokens, on pairs of SMs (``gemm_tcgen05_2cta.cu``)."""
    global _pair_lib
    if _pair_lib is None:
        l = load_module("gemm_pair", ["gemm_tcgen05_2cta.cu"])
        l.ib_gemm_pair.argtypes = [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                   _c_void_p]
        l.ib_gemm_pair.restype = _c_int
        lib()  # the SM count
        _pair_lib = l
    return _pair_lib


def _error_word(device) -> torch.Tensor:
    """The word for calls that bring none (a kernel run on its own, outside a
    model step); a model's products always bring their engine's word."""
    ws = _workspaces.get(device)
    if ws is None:
        ws = {"err": core.new_error_word(device)}
        _workspaces[device] = ws
    return ws["err"]


def choose_splits(T: int, N: int, K: int, sm_count: int) -> int:
    """Slices of K (1..8, the CTAs of one cluster).  Two CTAs fit an SM; the
    largest slice count is taken whose grid still fits one round with some room
    for the placement of whole clusters (measured on the 8B shapes: 48 tiles x 5
    and 32 tiles x 8 run in one round, 48 x 6 does not), each slice keeping at
    least four blocks of 64 k."""
    bn = lib().ib_gemm_tc_token_tile(T)
    tiles = -(-N // BM) * -(-T // bn)
    kblocks = -(-K // BK)
    room = int(0.87 * 2 * sm_count)
    best = 1
    for s in range(2, 9):
        if tiles * s <= room and kblocks // s >= 4:
            best = s
    return best


def eligible(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and out.dtype in (torch.bfloat16, torch.float32)
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.shape[1] % 8 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: Optional[int] = None,
            err: Optional[torch.Tensor] = None, swiglu: bool = False) -> None:
    """Runs the tcgen05 kernel; raises KernelError if the operands do not fit it.
    ``swiglu``: ``w`` holds, per 128 rows, 64 gate rows then their 64 up rows, and
    ``out`` [T, N/2] receives silu(gate) * up (at most 64 tokens)."""
    core.require_cuda(x, w, out)
    T, K = x.shape
    N = w.shape[0]
    if splits is None:
        splits = choose_splits(T, N, K, POLICY["sm_count"])
    code = lib().ib_gemm_tc(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                            out.stride(0), 1 if out.dtype == torch.float32 else 0, T, N, K, splits,
                            1 if swiglu else 0, (err if err is not None else _error_word(x.device)).data_ptr(),
                            core.stream_ptr(x))
    core.check(code, "gemm_tc")


@functools.lru_cache(maxsize=256)
def choose_pair_tiling(T: int, N: int, sm_count: int, swiglu: bool = False) -> Tuple[int, int, int]:
    """How ``gemm_pair`` cuts the weight rows: ``(bn_a, cols_a, bn_b)`` = ``cols_a``
    columns of tiles ``bn_a`` rows wide, then the rest in columns ``bn_b`` wide.
    The pairs of SMs take the tiles in turn, so the time is that of the pair with
    the most work; a tile costs its width plus a constant (its token half is
    fetched and its first and last steps run whatever the width).  Mostly this
    ends in full-width tiles for the full rounds and a narrower last round."""
    pairs = max(sm_count // 2, 1)
    t_tiles = -(-T // 256)
    step = 128 if swiglu else 16
    widths = list(range(256, 127, -step))  # narrower tiles take as long as 128 rows
    best, best_cost = (256, -(-N // 256), 256), None
    for bn_a in (256,) if not swiglu else (256, 128):
        all_a = -(-N // bn_a)
        for cols_a in range(all_a, -1, -1):
            rest = N - cols_a * bn_a
            for bn_b in (widths if rest > 0 else [bn_a]):
                tiles_a = cols_a * t_tiles
                tiles_b = -(-rest // bn_b) * t_tiles if rest > 0 else 0
                total = tiles_a + tiles_b
                cost = 0
                # the pairs that matter: the first, and those around the region's and the list's end
                for pr in {0, (tiles_a - 1) % pairs, tiles_a % pairs, (total - 1) % pairs, pairs - 1}:
                    if pr >= total:
                        continue
                    n_all = -(-(total - pr) // pairs)
                    n_a = -(-(tiles_a - pr) // pairs) if pr < tiles_a else 0
                    cost = max(cost, n_a * (bn_a + PAIR_TILE_OVERHEAD) + (n_all - n_a) * (bn_b + PAIR_TILE_OVERHEAD))
                if best_cost is None or cost < best_cost:
                    best, best_cost = (bn_a, cols_a, bn_b), cost
    return best


def choose_token_group(T: int, K: int) -> int:
    """Token tiles (of 256) per group in ``gemm_pair``.  The pairs of SMs walk
    the tiles of one group, all weight columns, before the next group, so what a
    round of tiles reads of the tokens is one group's rows: ``group x 256 x K``
    values, kept under ``pair_group_bytes`` so that they stay in L2 beside the
    streamed weights.  (8,192 tokens as one group: the gate/up product runs at
    1,270 TFLOP/s, the down product, whose token operand is 235 MB, at 1,330,
    against 1,530 and 1,440 at 4,096 tokens.)  Groups are evened out."""
    t_tiles = -(-T // 256)
    most = max(2, min(POLICY["pair_group_max_tiles"], POLICY["pair_group_bytes"] // (512 * max(K, 1))))
    groups = -(-t_tiles // most)
    return -(-t_tiles // groups)


def gemm_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
              err: Optional[torch.Tensor] = None, swiglu: bool = False,
              tiling: Optional[Tuple[int, int, int]] = None, token_group: Optional[int] = None) -> None:
    """The product for many tokens: tiles of 256 tokens x up to 256 weight rows,
    each computed by two SMs as one (tcgen05 ``cta_group::2``); bf16 out.
    ``swiglu`` as in ``gemm_tc``, for any number of tokens."""
    core.require_cuda(x, w, out)
    T, K = x.shape
    N = w.shape[0]
    bn_a, cols_a, bn_b = tiling or choose_pair_tiling(T, N, POLICY["sm_count"], swiglu)
    code = pair_lib().ib_gemm_pair(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                   out.stride(0), T, N, K, 1 if swiglu else 0, bn_a, cols_a, bn_b,
                                   token_group or choose_token_group(T, K), POLICY["sm_count"],
                                   (err if err is not None else _error_word(x.device)).data_ptr(),
                                   core.stream_ptr(x))
    core.check(code, "gemm_pair")


def route(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None) -> bool:
    """Takes a product or leaves it to the library.  ``auto``: up to
    ``max_tokens`` tokens go to the kernel that streams the weights once, prompts
    whose length suits its tiles to the kernel on pairs of SMs (inside a model
    step it is ahead of the library, whose kernels do not let their successor
    start under their tail), the rest to the library; ``all``: every product."""
    mode = POLICY["mode"]
    if mode in ("none", "cublas", "library") or not eligible(x, w, out):
        return False
    T = x.shape[0]
    if T > POLICY["max_tokens"]:
        if (pair_suits(T) and out.dtype == torch.bfloat16 and out.stride(0) % 8 == 0
                and out.data_ptr() % 16 == 0):
            gemm_pair(x, w, out, err=err)
            return True
        if mode != "all":
            return False
    gemm_tc(x, w, out, err=err)
    return True


def swiglu_route(x: torch.Tensor, w_interleaved: torch.Tensor, out: torch.Tensor,
                 err: Optional[torch.Tensor] = None) -> bool:
    """The gate/up product with SiLU(gate) * up applied in its epilogue, when
    the policy and the operands allow; ``out`` is [T, I].  Up to 64 tokens go to
    the kernel that streams the weights once (decode), prompts to the kernel on
    pairs of SMs when their length suits its tiles (``pair_suits``)."""
    mode = POLICY["mode"]
    if mode in ("none", "cublas", "library"):
        return False
    if w_interleaved.shape[0] % 128 or out.dtype != torch.bfloat16:
        return False
    if not eligible(x, w_interleaved, out) or out.stride(0) % 8 or out.data_ptr() % 16:
        return False
    T = x.shape[0]
    if T <= min(POLICY["max_tokens"], 64):
        gemm_tc(x, w_interleaved, out, splits=1, swiglu=True, err=err)
        return True
    if pair_suits(T, fused_activation=True):
        gemm_pair(x, w_interleaved, out, swiglu=True, err=err)
        return True
    return False


def error_flags(device) -> int:
    ws = _workspaces.get(torch.device(device))
    return int(ws["err"].item()) if ws else 0
