"""Times one kernel of the package at given sizes and reports what it moves or
computes against the machine's measured peaks.  Meant for profiling: run it
plain to get the number, or under ``ncu --clock-control none -k regex:<kernel> -c 3`` for
counters (without that flag ncu locks the clocks of a GPU that others share).

    python -m infernum_b200.cli.kernel_bench attention-decode --batch 64 --kv-len 1100
    python -m infernum_b200.cli.kernel_bench attention-prefill --tokens 2048
    python -m infernum_b200.cli.kernel_bench attention-prefill --tokens 512 --prefix 3584
    python -m infernum_b200.cli.kernel_bench gemm --tokens 8 --n 4096 --k 4096
    python -m infernum_b200.cli.kernel_bench norm --tokens 2048 --hidden 4096
    python -m infernum_b200.cli.kernel_bench rope --tokens 2048
    python -m infernum_b200.cli.kernel_bench silu --tokens 2048 --intermediate 14336

Default sizes are those of the Llama-3.1-8B shape.  Inputs rotate through
several copies so that every timed launch reads from HBM, not from L2.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
from types import SimpleNamespace
from typing import Callable, List

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            return json.load(fh)
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def _time(fns: List[Callable[[], None]], reps: int, warmup: int, graph: bool = True) -> float:
    """Mean microseconds per call, cycling through ``fns``.  With ``graph`` the
    launches are recorded once in a CUDA graph and the replay is timed, so that
    short kernels are not measured at the speed of the host."""
    import torch

    for i in range(max(warmup, len(fns))):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(reps):
                fns[i % len(fns)]()
        g.replay()
        torch.cuda.synchronize()
        start.record()
        g.replay()
        end.record()
    else:
        start.record()
        for i in range(reps):
            fns[i % len(fns)]()
        end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1000.0 / reps


def _attention_case(batch, rows, kv_len, nh, nkv, hd, page_size, device):
    """``batch`` requests of ``kv_len`` tokens whose last ``rows`` are this step's."""
    import torch

    pages_per = -(-kv_len // page_size)
    n_pages = batch * pages_per
    g = torch.Generator(device="cpu").manual_seed(0)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    tables = perm.view(batch, pages_per).contiguous().to(device)
    kp = torch.randn(n_pages, nkv, page_size, hd, device=device).to(torch.bfloat16)
    vp = torch.randn(n_pages, nkv, page_size, hd, device=device).to(torch.bfloat16)
    q = torch.randn(batch * rows, (nh + 2 * nkv) * hd, device=device).to(torch.bfloat16)
    cu = [i * rows for i in range(batch + 1)]
    pos = [kv_len - rows + r for _ in range(batch) for r in range(rows)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)  # noqa: E731
    ctx = SimpleNamespace(
        n_rows=batch * rows, n_entries=batch, positions=i32(pos),
        row_entry=i32([b for b in range(batch) for _ in range(rows)]), cu_rows=i32(cu),
        q_start=i32([kv_len - rows] * batch), host_cu_rows=cu, max_rows_per_entry=rows,
        max_kv_len=kv_len, scratch={})
    return q, kp, vp, tables, ctx


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("kernel", choices=["attention-decode", "attention-prefill", "gemm", "norm", "rope", "silu"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--kv-len", type=int, default=1100)
    ap.add_argument("--prefix", type=int, default=0, help="attention-prefill: cached tokens before the portion")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=14336)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--splits", type=int, default=0, help="force a slice count (attention-decode, attention-prefill, gemm)")
    ap.add_argument("--reps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--library", action="store_true", help="gemm: time the library product instead")
    ap.add_argument("--token-group", type=int, default=0,
                    help="gemm --pair: token tiles of 256 per group (default: chosen from the sizes)")
    ap.add_argument("--bn", type=int, default=0, help="gemm --pair: force the tile's weight rows")
    ap.add_argument("--swiglu", action="store_true", help="gemm --pair: SiLU(gate) * up in the epilogue")
    ap.add_argument("--pair", action="store_true", help="gemm: the kernel on pairs of SMs (many tokens)")
    ap.add_argument("--no-tma", action="store_true", help="attention-decode: fetch keys and values with cp.async")
    ap.add_argument("--no-graph", action="store_true", help="launch from the host instead of replaying a graph")
    args = ap.parse_args(argv)

    import torch

    from ..ops import attention_fast, core, gemm_tc
    from ..parts.base import Runtime

    dev = torch.device("cuda:0")
    peaks = _peaks()
    rt = Runtime(dev, torch.bfloat16, err=core.new_error_word(dev),
                 options={"sm_count": torch.cuda.get_device_properties(0).multi_processor_count})
    nh, nkv, hd = args.heads, args.kv_heads, args.head_dim
    if args.no_tma:
        rt.options["split_copy"] = "cp.async"
    out = {"kernel": args.kernel}

    if args.kernel in ("attention-decode", "attention-prefill"):
        decode = args.kernel == "attention-decode"
        batch = args.batch if decode else 1
        rows = 1 if decode else args.tokens
        # a prompt portion may come after a cached prefix: --prefix tokens already in the cache
        kv_len = args.kv_len if decode else args.tokens + args.prefix
        cases = [_attention_case(batch, rows, kv_len, nh, nkv, hd, args.page_size, dev)
                 for _ in range(2 if decode else 1)]
        outs = torch.empty(batch * rows, nh * hd, dtype=torch.bfloat16, device=dev)
        scale = 1.0 / math.sqrt(hd)
        fns = []
        for q, kp, vp, tables, ctx in cases:
            if decode and args.splits:
                ctx.attention_mode = (2, args.splits)
            if not decode and args.splits:
                ctx.prompt_splits = args.splits
            fns.append(lambda q=q, kp=kp, vp=vp, tables=tables, ctx=ctx: attention_fast.run(
                q, kp, vp, outs, ctx, tables, nh, scale, 0, rt))
        us = _time(fns, args.reps, args.warmup, not args.no_graph)
        if decode:
            nbytes = batch * kv_len * nkv * hd * 2 * 2
            out.update(batch=batch, kv_len=kv_len, us=us, gbs=nbytes / us / 1e3,
                       frac_of_hbm=nbytes / us / 1e3 / peaks["hbm_gbs"])
        else:
            flops = 4.0 * nh * hd * (rows * (rows + 1) / 2 + rows * args.prefix)
            out.update(tokens=rows, prefix=args.prefix, us=us, tflops=flops / us / 1e6,
                       frac_of_bf16=flops / us / 1e6 / peaks["bf16_tflops"])
    elif args.kernel == "gemm":
        T, N, K = args.tokens, args.n, args.k
        copies = max(2, int(300e6 / (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device=dev).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(T, K, device=dev).to(torch.bfloat16)
        o = torch.empty(T, N // 2 if args.swiglu else N, dtype=torch.bfloat16, device=dev)
        gemm_tc.POLICY["sm_count"] = rt.options["sm_count"]
        if args.library:
            fns = [lambda w=w: torch.mm(x, w.t(), out=o) for w in ws]
        elif args.pair:
            fns = [lambda w=w: gemm_tc.gemm_pair(x, w, o, err=rt.err, swiglu=args.swiglu,
                                                 tiling=(args.bn, 1 << 20, args.bn) if args.bn else None,
                                                 token_group=args.token_group or None)
                   for w in ws]
        else:
            fns = [lambda w=w: gemm_tc.gemm_tc(x, w, o, splits=args.splits or None) for w in ws]
        us = _time(fns, args.reps, args.warmup, not args.no_graph)
        nbytes, flops = N * K * 2 + T * K * 2 + T * N * 2, 2.0 * T * N * K
        out.update(tokens=T, n=N, k=K, us=us, gbs=nbytes / us / 1e3, tflops=flops / us / 1e6,
                   frac_of_hbm=nbytes / us / 1e3 / peaks["hbm_gbs"],
                   frac_of_bf16=flops / us / 1e6 / peaks["bf16_tflops"],
                   library=bool(args.library))
    elif args.kernel == "norm":
        T, H = args.tokens, args.hidden
        n = max(2, int(300e6 / (T * H * 12)) + 1)
        res = [torch.randn(T, H, device=dev) for _ in range(n)]
        delta = [torch.randn(T, H, device=dev).to(torch.bfloat16) for _ in range(n)]
        w = torch.ones(H, dtype=torch.bfloat16, device=dev)
        o = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        fns = [lambda r=r, d=d: core.add_rmsnorm(r, d, w, 1e-5, o) for r, d in zip(res, delta)]
        us = _time(fns, args.reps, args.warmup, not args.no_graph)
        nbytes = T * H * (4 + 2 + 4 + 2)
        out.update(tokens=T, hidden=H, us=us, gbs=nbytes / us / 1e3,
                   frac_of_hbm=nbytes / us / 1e3 / peaks["hbm_gbs"])
    elif args.kernel == "rope":
        T = args.tokens
        width = (nh + 2 * nkv) * hd
        qkv = torch.randn(T, width, device=dev).to(torch.bfloat16)
        ps = args.page_size
        pages = -(-T // ps)
        kp = torch.zeros(pages, nkv, ps, hd, dtype=torch.bfloat16, device=dev)
        vp = torch.zeros_like(kp)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        ent = torch.zeros(T, dtype=torch.int32, device=dev)
        tables = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        inv = torch.rand(hd // 2, device=dev)
        fns = [lambda: core.rope_append(qkv, pos, inv, hd, nh, nkv, hd, ent, tables, kp, vp, rt.err)]
        us = _time(fns, args.reps, args.warmup, not args.no_graph)
        nbytes = T * ((nh + nkv) * hd * 2 * 2 + nkv * hd * 2 + 2 * nkv * hd * 2)
        out.update(tokens=T, us=us, gbs=nbytes / us / 1e3, frac_of_hbm=nbytes / us / 1e3 / peaks["hbm_gbs"])
    elif args.kernel == "silu":
        T, I = args.tokens, args.intermediate
        n = max(2, int(300e6 / (T * I * 6)) + 1)
        xs = [torch.randn(T, 2 * I, device=dev).to(torch.bfloat16) for _ in range(n)]
        o = torch.empty(T, I, dtype=torch.bfloat16, device=dev)
        fns = [lambda x=x: core.silu_mul(x, o) for x in xs]
        us = _time(fns, args.reps, args.warmup, not args.no_graph)
        nbytes = T * I * 6
        out.update(tokens=T, intermediate=I, us=us, gbs=nbytes / us / 1e3,
                   frac_of_hbm=nbytes / us / 1e3 / peaks["hbm_gbs"])
    flags = int(rt.err.item())
    out["error_flags"] = flags
    print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in out.items()}))
    return 1 if flags else 0


if __name__ == "__main__":
    sys.exit(main())
