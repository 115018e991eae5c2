"""Trace replay: feeds given token ids through a model step by step and writes
the logits at the wanted places.  It samples nothing and schedules nothing -
the trace is the schedule - and it has no forward pass, cache or loader of its
own: it drives the model, step function, cache manager and kernels that
generation uses.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
``entries``: for each request its next tokens and the places among them whose
logits are wanted; all entries of a step are one batch.  ``end``: requests that
are finished after this step; their pages and slot are given back.  For a step
that wants something, DIR/<step>.f32 holds the logits [wanted, vocab] as
little-endian float32 in the order of the entries and of ``want``.  After every
step a line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import IO, List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                 formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels and precisions serving uses; "
                         "float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each request's count "
                         "rounded up to a multiple of 64; the page pool is made for this many")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (divides 64)")
    ap.add_argument("--max-live", type=int, default=8, help="request slots")
    ap.add_argument("--device", default="cuda:0")
    return ap


def replay(args, stdin: IO[str], stdout: IO[str]) -> int:
    import torch

    from ..cache import CacheManager
    from ..engine.step import ModelRunner, StepEntry
    from ..loading import load_model

    if args.page_size <= 0 or 64 % args.page_size:
        raise SystemExit("--page-size must divide 64")
    os.makedirs(args.out, exist_ok=True)
    model = load_model(args.model, dtype=args.dtype, device=args.device)
    num_pages = max(1, (args.max_tokens + 63) // 64) * (64 // args.page_size)
    cache = CacheManager(model.cache_needs(), page_size=args.page_size, num_pages=num_pages,
                         max_requests=args.max_live, dtype=model.rt.dtype, device=model.rt.device)
    runner = ModelRunner(model, cache, max_rows=max(args.max_tokens, 64),
                         max_entries=args.max_live)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries: List[StepEntry] = []
        for ent in rec.get("entries", []):
            rid = ent["id"]
            rc = cache.get(rid) if cache.has(rid) else cache.admit(rid)
            entries.append(StepEntry(rc, ent["tokens"], ent.get("want", [])))
        if entries:
            logits = runner.step(entries)
            runner.check_errors()
            if logits is not None:
                arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{rec['step']}.f32"))
        for rid in rec.get("end", []):
            if cache.has(rid):
                cache.release(cache.get(rid))
        stdout.write(f"done {rec['step']}\n")
        stdout.flush()
    return 0


def main(argv: Optional[List[str]] = None, stdin: Optional[IO[str]] = None,
         stdout: Optional[IO[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    return replay(args, stdin or sys.stdin, stdout or sys.stdout)


if __name__ == "__main__":
    sys.exit(main())
