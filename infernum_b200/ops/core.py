"""Python side of the ``core`` kernel module: argument checks and ctypes calls.

Every function here launches hand-written CUDA on the current stream of the
tensor's device.  There is no CPU or library fallback: a tensor that is not on
a CUDA device, or a missing/unbuildable extension, raises ``KernelError``.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..csrc.build import load_module
from ..errors import KernelError

CORE_SOURCES = ["elementwise.cu", "attention_plain.cu", "gemm_plain.cu", "sampling.cu"]

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_void_p = ctypes.c_void_p
_c_ll = ctypes.c_longlong

FLAG_BAD_TOKEN = 1
FLAG_BAD_PAGE = 2
FLAG_WAIT_TIMEOUT = 4
# beside FLAG_WAIT_TIMEOUT, bit 8 + i says which wait gave up (common.cuh: IB_SITE_*)
TIMEOUT_SITES = ["product for few tokens: producer", "product for few tokens: MMA issuer",
                 "product for few tokens: epilogue", "product on SM pairs: producer",
                 "product on SM pairs: MMA issuer", "product on SM pairs: epilogue",
                 "prompt attention: producer", "prompt attention: MMA issuer", "prompt attention: softmax",
                 "prompt attention: shared memory window misplaced", "decode attention: producer",
                 "decode attention: computing warps"]


def describe_flags(flags: int) -> str:
    what = [name for bit, name in ((FLAG_BAD_TOKEN, "token id outside the vocabulary"),
                                   (FLAG_BAD_PAGE, "block-table entry outside the pool"),
                                   (FLAG_WAIT_TIMEOUT, "a device-side wait ran out")) if flags & bit]
    sites = [name for i, name in enumerate(TIMEOUT_SITES) if flags & (1 << (8 + i))]
    return "; ".join(what) + (" (" + ", ".join(sites) + ")" if sites else "")

_ERR_NAMES = {-1: "bad argument", -2: "unsupported configuration", -3: "size beyond the kernel's maximum",
              -4: "per-device set-up failed"}

_lib = None


def core_lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = load_module("core", CORE_SOURCES)
        lib.ib_wait_probe.argtypes = [_c_void_p, _c_ll, _c_int, _c_void_p]
        lib.ib_wait_probe.restype = _c_int
        lib.ib_step_fence.argtypes = [_c_void_p]
        lib.ib_step_fence.restype = _c_int
        lib.ib_embed.argtypes = [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int,
                                 _c_void_p, _c_void_p]
        lib.ib_add_rmsnorm.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                                       _c_void_p, _c_int, _c_int, _c_float, _c_int, _c_void_p]
        lib.ib_residual_add.argtypes = [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p]
        lib.ib_rope_append.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                       _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                       _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                       _c_void_p]
        lib.ib_silu_mul.argtypes = [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_attention_plain.argtypes = [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                           _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                           _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                           _c_float, _c_void_p, _c_void_p]
        lib.ib_gemm_plain.argtypes = [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int,
                                      _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p]
        lib.ib_argmax.argtypes = [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_ll,
                                  _c_void_p]
        lib.ib_sample.argtypes = [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                                  _c_void_p, _c_void_p]
        lib.ib_decode_advance.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                          _c_void_p]
        lib.ib_feed_tokens.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p,
                                       _c_void_p]
        for fn in ("ib_decode_advance", "ib_feed_tokens", "ib_embed", "ib_add_rmsnorm", "ib_residual_add", "ib_rope_append",
                   "ib_silu_mul", "ib_attention_plain", "ib_gemm_plain", "ib_argmax", "ib_sample"):
            getattr(lib, fn).restype = _c_int
        _lib = lib
    return _lib


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


_step_stream: Optional[int] = None  # the stream of the step being launched, looked up once per step


def stream_ptr(t: torch.Tensor) -> int:
    if _step_stream is not None:
        return _step_stream
    return torch.cuda.current_stream(t.device).cuda_stream


class step_stream:
    """While a model step is being launched, every kernel goes to the stream that
    was current at its start; looking it up for each launch costs as much as a
    small launch itself."""

    def __init__(self, device):
        self.device = device

    def __enter__(self):
        global _step_stream
        self.previous = _step_stream
        _step_stream = torch.cuda.current_stream(self.device).cuda_stream
        return self

    def __exit__(self, *exc):
        global _step_stream
        _step_stream = self.previous
        return False


LAUNCHES = 0  # kernels of this package launched so far (benchmarks report the count)

# ---------------------------------------------------------------------------
# INFERNUM_PROFILE=1: the device time of every operation, summed per operation
# and printed as a table when the process ends (the reference does this for its
# CPU executor: infernum-cpu/src/executor.rs:24-62).  A CUDA event is recorded
# before and behind every launch.  For the time between the two to be the
# operation's, the kernels must not overlap and must be launched one by one:
# in this mode programmatic dependent launch is off and the engine replays no
# recordings.  What the table shows is therefore not what a step costs in
# service, where kernels start under their predecessor's tail: it shows where
# the time goes.  A kernel that starts on an idle stream pays its launch
# (some 10 to 15 us between the two events even for the smallest kernel), and
# the first call of a library product pays the library's set-up: read the
# shares of the large operations here, and a kernel's own duration from
# ``ncu`` or ``python -m infernum_b200.cli.kernel_bench``.
# ---------------------------------------------------------------------------
PROFILE = os.environ.get("INFERNUM_PROFILE", "0") not in ("", "0")
_profile_marks: list = []  # (operation, event before, event after), in launch order
_profile_totals: dict = {}  # operation -> [calls, microseconds]
_profile_open = None  # the event before the operation being launched


def _profile_event():
    ev = torch.cuda.Event(enable_timing=True)
    ev.record(torch.cuda.current_stream() if _step_stream is None else torch.cuda.ExternalStream(_step_stream))
    return ev


def profile_begin() -> None:
    """The start of an operation (profile mode only): every wrapper passes here
    on its way in (``require_cuda``); ``profile_mark`` closes it."""
    global _profile_open
    if PROFILE and _profile_open is None:
        _profile_open = _profile_event()


def profile_mark(what: str) -> None:
    """The end of operation ``what`` on the current stream (profile mode only).
    Its time runs from ``profile_begin``, or from the end of the operation
    before it when one wrapper launches two kernels."""
    global _profile_open
    if not PROFILE:
        return
    after = _profile_event()
    before = _profile_open if _profile_open is not None else (_profile_marks[-1][2] if _profile_marks else after)
    _profile_open = None
    _profile_marks.append((what, before, after))
    if len(_profile_marks) >= 20000:
        profile_collect()


def profile_collect() -> dict:
    """Folds the marks so far into the totals and returns them: operation -> [calls, microseconds]."""
    if _profile_marks:
        torch.cuda.synchronize()
        for what, before, after in _profile_marks:
            row = _profile_totals.setdefault(what, [0, 0.0])
            row[0] += 1
            row[1] += before.elapsed_time(after) * 1000.0
        del _profile_marks[:]
    return _profile_totals


def profile_report(file=None) -> str:
    """The table of ``profile_collect``; printed to ``file`` when given."""
    totals = profile_collect()
    whole = sum(v[1] for v in totals.values()) or 1.0
    lines = [f"{'operation':28s} {'calls':>8s} {'total ms':>10s} {'mean us':>9s} {'share':>7s}"]
    for what, (calls, us) in sorted(totals.items(), key=lambda kv: -kv[1][1]):
        lines.append(f"{what:28s} {calls:8d} {us / 1000:10.2f} {us / max(calls, 1):9.2f} {100 * us / whole:6.1f}%")
    text = "\n".join(lines)
    if file is not None:
        print(text, file=file)
    return text


if PROFILE:
    import atexit
    import sys as _sys

    atexit.register(lambda: profile_report(_sys.stderr) if (_profile_marks or _profile_totals) else None)


def check(code: int, what: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        if PROFILE:
            profile_mark(what)
        return
    if code < 0:
        raise KernelError(f"{what}: kernel refused its arguments ({_ERR_NAMES.get(code, code)})")
    raise KernelError(f"{what}: CUDA launch failed with error {code}")


def require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    if PROFILE:
        profile_begin()
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError(
                "infernum_b200 kernels run on a CUDA device only; got a tensor on "
                f"{t.device} (there is no CPU path)"
            )


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _int32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous int32 tensor")


def new_error_word(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def wait_probe(err: torch.Tensor, limit_ms: float, site: int) -> None:
    """Runs a kernel whose one wait nothing ends: after ``limit_ms`` it sets the
    time-out flag with the bit of ``site`` in ``err`` and returns.  For testing
    that a wait that runs out is reported and leaves the device usable."""
    require_cuda(err)
    check(core_lib().ib_wait_probe(err.data_ptr(), int(limit_ms * 1e6), int(site), stream_ptr(err)),
          "wait_probe")


def step_fence(device) -> None:
    """The first launch of a step: an empty kernel launched the ordinary way, so
    that no kernel of the step starts before everything earlier in the stream -
    the copies and kernels that wrote the step's positions and tables - is
    complete (the package's other kernels start under their predecessor's tail
    and read those early)."""
    check(core_lib().ib_step_fence(torch.cuda.current_stream(device).cuda_stream), "step_fence")


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor) -> None:
    """out[t, :] = table[ids[t], :] into a float32 residual stream."""
    require_cuda(ids, table, out, err)
    _int32(ids, "ids")
    n = ids.numel()
    V, H = table.shape
    if out.dtype != torch.float32 or out.shape != (n, H) or not out.is_contiguous():
        raise KernelError(f"embed: out must be contiguous float32 [{n}, {H}]")
    if not table.is_contiguous():
        raise KernelError("embed: table must be contiguous")
    check(core_lib().ib_embed(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype),
                              out.data_ptr(), n, H, V, err.data_ptr(), stream_ptr(out)), "embed")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: torch.Tensor, row_idx: Optional[torch.Tensor] = None,
                write_residual: bool = True) -> None:
    """residual (+)= delta; out = rmsnorm(residual) * weight, in 32-bit.

    With ``row_idx`` only those rows are normed, ``out`` is compact and the
    residual is left as it was."""
    require_cuda(residual, delta, weight, out, row_idx)
    N, H = residual.shape
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError("add_rmsnorm: residual must be contiguous float32")
    n_out = N if row_idx is None else row_idx.numel()
    _int32(row_idx, "row_idx")
    if row_idx is not None:
        write_residual = False
    if out.shape != (n_out, H) or not out.is_contiguous():
        raise KernelError(f"add_rmsnorm: out must be contiguous [{n_out}, {H}]")
    if delta is not None and (delta.shape != residual.shape or delta.dtype != out.dtype
                              or not delta.is_contiguous()):
        raise KernelError("add_rmsnorm: delta must match the residual's shape and out's dtype")
    if weight.shape != (H,) or not weight.is_contiguous():
        raise KernelError(f"add_rmsnorm: weight must be [{H}]")
    check(core_lib().ib_add_rmsnorm(residual.data_ptr(), _ptr(delta), weight.data_ptr(),
                                    dtype_code(weight.dtype), out.data_ptr(),
                                    dtype_code(out.dtype), _ptr(row_idx), n_out, H, float(eps),
                                    1 if write_residual else 0, stream_ptr(out)), "add_rmsnorm")


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    require_cuda(residual, delta)
    if residual.dtype != torch.float32 or residual.shape != delta.shape \
            or not residual.is_contiguous() or not delta.is_contiguous():
        raise KernelError("residual_add: shapes must match, residual float32, both contiguous")
    check(core_lib().ib_residual_add(residual.data_ptr(), delta.data_ptr(),
                                     dtype_code(delta.dtype), residual.numel(),
                                     stream_ptr(residual)), "residual_add")


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                rotary_dim: int, n_heads: int, n_kv_heads: int, head_dim: int,
                row_entry: Optional[torch.Tensor], block_tables: Optional[torch.Tensor],
                k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                err: torch.Tensor) -> None:
    """Rotate q and k of ``qkv`` in place; with pools, store k and v in the pages."""
    require_cuda(qkv, positions, inv_freq, row_entry, block_tables, k_pool, v_pool, err)
    _int32(positions, "positions")
    _int32(row_entry, "row_entry")
    _int32(block_tables, "block_tables")
    N = qkv.shape[0]
    if qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelError("rope_append: qkv must be 2-D with unit inner stride")
    write_kv = k_pool is not None
    page_size = num_pages = max_blocks = 0
    if write_kv:
        if k_pool.shape != v_pool.shape or k_pool.dtype != qkv.dtype or v_pool.dtype != qkv.dtype \
                or not k_pool.is_contiguous() or not v_pool.is_contiguous():
            raise KernelError("rope_append: pools must be contiguous, alike and of qkv's dtype")
        num_pages, nkv_pool, page_size, hd_pool = k_pool.shape
        if nkv_pool != n_kv_heads or hd_pool != head_dim:
            raise KernelError("rope_append: pool shape does not match the head counts")
        max_blocks = block_tables.shape[1]
    need = (n_heads + (2 * n_kv_heads if write_kv else n_kv_heads)) * head_dim
    if qkv.shape[1] < need:
        raise KernelError(f"rope_append: qkv rows hold {qkv.shape[1]} values, need {need}")
    if rotary_dim > 0 and (inv_freq is None or inv_freq.dtype != torch.float32
                           or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("rope_append: inv_freq must be float32 [rotary_dim / 2]")
    check(core_lib().ib_rope_append(qkv.data_ptr(), dtype_code(qkv.dtype), qkv.stride(0),
                                    positions.data_ptr(), _ptr(row_entry), _ptr(block_tables),
                                    max_blocks, _ptr(inv_freq), _ptr(k_pool), _ptr(v_pool), N,
                                    n_heads, n_kv_heads, head_dim, rotary_dim, page_size,
                                    num_pages, 1 if write_kv else 0, err.data_ptr(),
                                    stream_ptr(qkv)), "rope_append")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, block: Optional[int] = None) -> None:
    """out = silu(gate) * up for rows [N, 2I].  ``block`` says where gates and
    ups sit in a row: None for [all gates | all ups], else pieces of ``block``
    gates followed by their ``block`` ups."""
    require_cuda(gate_up, out)
    N, two_i = gate_up.shape
    if two_i % 2 or out.shape != (N, two_i // 2) or out.dtype != gate_up.dtype \
            or not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError("silu_mul: gate_up [N, 2I] and out [N, I] must be contiguous, same dtype")
    I = two_i // 2
    blk = I if block is None else int(block)
    if blk <= 0 or I % blk:
        raise KernelError(f"silu_mul: block {blk} does not divide the width {I}")
    check(core_lib().ib_silu_mul(gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), N, I,
                                 blk, stream_ptr(out)), "silu_mul")


def attention_plain(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    out: torch.Tensor, positions: torch.Tensor, row_entry: torch.Tensor,
                    block_tables: torch.Tensor, n_heads: int, scale: float, window: int,
                    err: torch.Tensor) -> None:
    """Causal attention of each row over its request's pages (32-bit arithmetic).

    ``q`` is [N, >= n_heads*hd] (a view into the qkv rows is fine), ``out`` is
    [N, n_heads*hd]; pools are [pages, kv_heads, page_size, hd]."""
    require_cuda(q, k_pool, v_pool, out, positions, row_entry, block_tables, err)
    _int32(positions, "positions")
    _int32(row_entry, "row_entry")
    _int32(block_tables, "block_tables")
    num_pages, nkv, page_size, hd = k_pool.shape
    N = q.shape[0]
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] < n_heads * hd \
            or out.shape[1] < n_heads * hd:
        raise KernelError("attention_plain: q/out rows are too short or not unit-stride")
    if not (q.dtype == k_pool.dtype == v_pool.dtype == out.dtype):
        raise KernelError("attention_plain: q, pools and out must share a dtype")
    if n_heads % nkv:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {nkv} kv heads")
    check(core_lib().ib_attention_plain(q.data_ptr(), q.stride(0), k_pool.data_ptr(),
                                        v_pool.data_ptr(), out.data_ptr(), out.stride(0),
                                        dtype_code(q.dtype), positions.data_ptr(),
                                        row_entry.data_ptr(), block_tables.data_ptr(),
                                        block_tables.shape[1], N, n_heads, nkv, hd, page_size,
                                        num_pages, int(window), float(scale), err.data_ptr(),
                                        stream_ptr(q)), "attention_plain")


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T with 32-bit fused multiply-adds in k order."""
    require_cuda(a, w, out)
    M, K = a.shape
    N, K2 = w.shape
    if K != K2 or out.shape != (M, N):
        raise KernelError(f"gemm_plain: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_plain: inner strides must be 1")
    check(core_lib().ib_gemm_plain(a.data_ptr(), dtype_code(a.dtype), a.stride(0), w.data_ptr(),
                                   dtype_code(w.dtype), w.stride(0), out.data_ptr(),
                                   dtype_code(out.dtype), out.stride(0), M, N, K,
                                   stream_ptr(out)), "gemm_plain")


_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """Greedy selection per row: the largest logit, the lowest index among equals."""
    require_cuda(logits, out)
    _int32(out, "out")
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.numel() != R:
        raise KernelError("argmax: logits must be float32 [R, V], out int32 [R]")
    scratch_ptr, scratch_bytes = None, 0
    if V >= 16384:
        # partial results of the sliced kernel: 64 (value, index) pairs per row
        key = (logits.device, R)
        buf = _argmax_scratch.get(key)
        if buf is None:
            buf = torch.empty(R * 64 * 2, dtype=torch.int32, device=logits.device)
            _argmax_scratch[key] = buf
        scratch_ptr, scratch_bytes = buf.data_ptr(), buf.numel() * 4
    check(core_lib().ib_argmax(logits.data_ptr(), logits.stride(0), R, V, out.data_ptr(),
                               scratch_ptr, scratch_bytes, stream_ptr(logits)), "argmax")


SAMPLE_PARAM_FLOATS = 6  # temperature, top_p, penalty, u, n_recent (int bits), pad


def sample(logits: torch.Tensor, params: torch.Tensor, recent: Optional[torch.Tensor],
           out: torch.Tensor) -> None:
    """Temperature / nucleus / repetition-penalty sampling; ``params`` is a
    [R, 6] float32 tensor (see ``pack_sample_params``).  Logits are modified in
    place by the penalty."""
    require_cuda(logits, params, recent, out)
    _int32(out, "out")
    _int32(recent, "recent")
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with unit inner stride")
    if params.dtype != torch.float32 or params.shape != (R, SAMPLE_PARAM_FLOATS) \
            or not params.is_contiguous():
        raise KernelError("sample: params must be contiguous float32 [R, 6]")
    recent_ld = 0 if recent is None else recent.shape[1]
    check(core_lib().ib_sample(logits.data_ptr(), logits.stride(0), R, V, params.data_ptr(),
                               _ptr(recent), recent_ld, out.data_ptr(), stream_ptr(logits)),
          "sample")


def feed_tokens(tokens: torch.Tensor, src: torch.Tensor, selected: torch.Tensor,
                recent: Optional[torch.Tensor] = None, recent_pos: Optional[torch.Tensor] = None) -> None:
    """tokens[i] = selected[src[i]] where src[i] >= 0 (other rows keep theirs): the
    inputs of a step launched behind the step whose selection ``selected`` is.
    With ``recent`` [rows, width] and ``recent_pos`` [rows], the same token is
    also written to ``recent[i, recent_pos[i]]`` where that place is not
    negative (the row's recent tokens, for its repetition penalty)."""
    require_cuda(tokens, src, selected, recent, recent_pos)
    for t, name in ((tokens, "tokens"), (src, "src"), (selected, "selected"), (recent, "recent"),
                    (recent_pos, "recent_pos")):
        _int32(t, name)
    if src.numel() < tokens.numel():
        raise KernelError("feed_tokens: fewer sources than tokens")
    if recent is not None and (recent_pos is None or recent.dim() != 2 or recent.shape[0] < tokens.numel()
                               or recent_pos.numel() < tokens.numel()):
        raise KernelError("feed_tokens: the recent tokens need a row and a place per token")
    check(core_lib().ib_feed_tokens(tokens.data_ptr(), src.data_ptr(), selected.data_ptr(), selected.numel(),
                                    tokens.numel(), _ptr(recent), recent.shape[1] if recent is not None else 0,
                                    _ptr(recent_pos), stream_ptr(tokens)), "feed_tokens")


def decode_advance(tokens: torch.Tensor, selected: Optional[torch.Tensor], positions: torch.Tensor,
                   kv_len: torch.Tensor, slot_ids: Optional[torch.Tensor] = None, pad_slot: int = -1) -> None:
    """positions += 1, kv_len += 1, and tokens = selected when given; rows whose
    slot is ``pad_slot`` (they only fill up a batch bucket) are left alone."""
    require_cuda(tokens, selected, positions, kv_len, slot_ids)
    for t, name in ((tokens, "tokens"), (selected, "selected"), (positions, "positions"), (kv_len, "kv_len"),
                    (slot_ids, "slot_ids")):
        _int32(t, name)
    check(core_lib().ib_decode_advance(tokens.data_ptr(), _ptr(selected), positions.data_ptr(),
                                       kv_len.data_ptr(), _ptr(slot_ids), int(pad_slot), tokens.numel(),
                                       stream_ptr(tokens)),
          "decode_advance")
