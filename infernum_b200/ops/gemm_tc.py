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
import os
from typing import Dict, Optional

import torch

from ..csrc.build import load_module
from . import core

_c_int, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong
_lib: Optional[ctypes.CDLL] = None
_workspaces: Dict[torch.device, dict] = {}

BM, BK = 128, 64

# Which products the kernel takes: "all", "none", or a largest token count.
POLICY = {"mode": os.environ.get("INFERNUM_GEMM", "auto"), "max_tokens": 64, "sm_count": 148}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        l = load_module("gemm_tc", ["gemm_tcgen05.cu"])
        l.ib_gemm_tc.argtypes = [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int,
                                 _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p]
        l.ib_gemm_tc.restype = _c_int
        l.ib_gemm_tc_token_tile.argtypes = [_c_int]
        l.ib_gemm_tc_token_tile.restype = _c_int
        _lib = l
    return _lib


def _error_word(device) -> torch.Tensor:
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


def route(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    mode = POLICY["mode"]
    if mode in ("none", "cublas", "library"):
        return False
    if mode == "auto" and x.shape[0] > POLICY["max_tokens"]:
        return False
    if not eligible(x, w, out):
        return False
    gemm_tc(x, w, out)
    return True


def swiglu_route(x: torch.Tensor, w_interleaved: torch.Tensor, out: torch.Tensor) -> bool:
    """The gate/up product with SiLU(gate) * up applied in its epilogue, when
    the policy and the operands allow; ``out`` is [T, I]."""
    mode = POLICY["mode"]
    if mode in ("none", "cublas", "library") or x.shape[0] > min(POLICY["max_tokens"], 64):
        return False
    if w_interleaved.shape[0] % 128 or out.dtype != torch.bfloat16:
        return False
    if not eligible(x, w_interleaved, out):
        return False
    gemm_tc(x, w_interleaved, out, splits=1, swiglu=True)
    return True


def error_flags(device) -> int:
    ws = _workspaces.get(torch.device(device))
    return int(ws["err"].item()) if ws else 0
