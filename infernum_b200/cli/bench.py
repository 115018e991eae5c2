"""``bench``: throughput of a model through the engine, in the manner of the
reference's example (infernum-examples/examples/bench.rs:72-158, 1035-1036):

    bench MODEL [N_GEN] [--dtype bf16|f32] [--graph | --graph-decode] [--cuda-graph-engine] [--gpus 1]

``MODEL`` is a model folder, or one of the shapes ``8b``, ``1b``, ``13b``,
``tinyA``, ``tinyB`` with random weights.  The default workload is the
reference's: an 8-token prompt, ``N_GEN`` (128) greedy tokens timed from the
host, and a 512-token prompt timed as prefill; it prints
``N tokens in S s = R tok/s``.  Two more workloads exercise the scheduler:

    --workload mixed      64 requests (``--requests``), prompt lengths uniform in
                          [16, 4096], prompts fed 512 tokens at a time beside the
                          decoding requests, 128 new tokens each, temperature 0.8
    --workload pressure   32 requests of 2,048 prompt + 512 greedy tokens with a
                          page pool too small for all of them, so that requests
                          are preempted and recomputed; every request's tokens
                          must equal its run alone

``--requests``, ``--prompt-len``, ``--new-tokens``, ``--num-blocks`` scale a
workload down; ``--layers`` cuts the number of layers of a random shape.
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import time
from typing import List, Optional

SHAPES = {
    "8b": {"num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32,
           "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
           "vocab_size": 128256, "rope_theta": 500000.0, "rms_norm_eps": 1e-5,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                            "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
           "tie_word_embeddings": False, "max_position_embeddings": 8192},
    "1b": {"num_hidden_layers": 16, "hidden_size": 2048, "num_attention_heads": 32,
           "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
           "vocab_size": 128256, "rope_theta": 500000.0, "rms_norm_eps": 1e-5,
           "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                            "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
           "tie_word_embeddings": True, "max_position_embeddings": 8192},
    "13b": {"num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40,
            "num_key_value_heads": 40, "head_dim": 128, "intermediate_size": 13824,
            "vocab_size": 32000, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
            "tie_word_embeddings": False, "max_position_embeddings": 4096},
    "tinyA": {"num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
              "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 176, "vocab_size": 256,
              "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
              "max_position_embeddings": 128},
    "tinyB": {"num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
              "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256, "vocab_size": 320,
              "rope_theta": 500000.0, "rms_norm_eps": 1e-6,
              "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                               "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
              "tie_word_embeddings": False, "max_position_embeddings": 256},
}


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="bench", description=__doc__,
                                 formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("model", help="model folder, or a shape name: " + ", ".join(SHAPES))
    ap.add_argument("n_gen", nargs="?", type=int, default=128, help="tokens to generate")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32", "bfloat16", "float32"])
    # the reference's mode switches (bench.rs:72-104).  It has several engines to choose from;
    # here there is one, which records and replays its steps, so two of them only say so.
    ap.add_argument("--graph", action="store_true",
                    help="prefill throughput: N_GEN tokens in a single forward pass")
    ap.add_argument("--graph-decode", action="store_true",
                    help="decode throughput: N_GEN tokens one by one (the default workload)")
    ap.add_argument("--cuda-graphs", action="store_true", help="accepted: steps are always recorded and replayed")
    ap.add_argument("--cuda-graph-engine", action="store_true", help="accepted: this is the only engine")
    ap.add_argument("--gpus", type=int, default=1, help="only 1: this engine runs on one GPU")
    ap.add_argument("--workload", default="single", choices=["single", "mixed", "pressure"])
    ap.add_argument("--requests", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--new-tokens", type=int, default=None)
    ap.add_argument("--num-blocks", type=int, default=None)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--solo-checks", type=int, default=None,
                    help="pressure: compare only so many requests with their run alone (preempted ones first)")
    ap.add_argument("--no-warmup", action="store_true",
                    help="mixed, pressure: time the first pass too (it records the steps' graphs)")
    ap.add_argument("--json", action="store_true", help="print one JSON object instead of text")
    return ap


def load(args):
    import infernum_b200 as ib

    dtype = {"bf16": "bfloat16", "f32": "float32"}.get(args.dtype, args.dtype)
    if args.model in SHAPES:
        cfg = dict(SHAPES[args.model], model_type="llama")
        if args.layers:
            cfg["num_hidden_layers"] = args.layers
        model = ib.random_model(cfg, seed=args.seed, dtype=dtype)
    else:
        model = ib.load_model(args.model, dtype=dtype)
    print(f"Model loaded: {len(model.layers)} layers, {model.spec.hidden_size} hidden, dtype={args.dtype}",
          file=sys.stderr)
    return model


def run_single(model, args) -> dict:
    import torch

    import infernum_b200 as ib

    vocab = model.spec.vocab_size
    prompt = [t % vocab for t in (1, 15043, 29892, 920, 526, 366, 2599, 13)]  # bench.rs:138
    n_gen = 8 if args.graph else args.n_gen
    prefill_tokens = min(args.n_gen if args.graph else 512, model.spec.max_position - 1)
    blocks = (max(prefill_tokens, len(prompt) + n_gen) + 1) // args.block_size + 4
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=1, block_size=args.block_size,
                                             num_blocks=blocks, max_prefill_tokens=max(2048, prefill_tokens),
                                             max_tokens_per_step=max(2048, prefill_tokens),
                                             max_model_len=max(prefill_tokens + 2, len(prompt) + n_gen + 1)))
    opts = ib.GenerateOptions(max_new_tokens=n_gen, ignore_eos=True)
    for _ in range(2):  # warm-up: a step's shape is recorded the second time it is met
        engine.generate(prompt, ib.GenerateOptions(max_new_tokens=8, ignore_eos=True))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    tokens = engine.generate(prompt, opts)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    rng = random.Random(args.seed)
    long_prompt = [rng.randrange(vocab) for _ in range(prefill_tokens)]
    one = ib.GenerateOptions(max_new_tokens=1, ignore_eos=True)
    for _ in range(2):  # warm-up: a step's shape is recorded the second time it is met
        engine.generate(long_prompt, one)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    engine.generate(long_prompt, one)
    torch.cuda.synchronize()
    dp = time.perf_counter() - t1
    return {"workload": "single", "generated": len(tokens), "seconds": dt, "decode_tok_s": len(tokens) / dt,
            "prefill_tokens": prefill_tokens, "prefill_tok_s": prefill_tokens / dp}


def run_mixed(model, args) -> dict:
    import torch

    import infernum_b200 as ib

    n_req = args.requests or 64
    new_tokens = args.new_tokens or 128
    max_prompt = args.prompt_len or 4096
    vocab = model.spec.vocab_size
    rng = random.Random(args.seed)
    lens = [rng.randint(min(16, max_prompt), max_prompt) for _ in range(n_req)]
    prompts = [[rng.randrange(vocab) for _ in range(n)] for n in lens]
    total = sum(lens) + n_req * new_tokens
    blocks = args.num_blocks or total // args.block_size + 2 * n_req
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=n_req, max_prefill_tokens=512,
                                             block_size=args.block_size, num_blocks=blocks,
                                             max_tokens_per_step=512 + n_req,
                                             max_model_len=max_prompt + new_tokens + 1))
    opts = [ib.GenerateOptions(max_new_tokens=new_tokens, ignore_eos=True,
                               sampling=ib.SamplingParams(temperature=0.8, top_p=1.0, seed=args.seed + i))
            for i in range(n_req)]
    if not args.no_warmup:
        # a step's shape is recorded the second time it is met and replayed from the third on
        for _ in range(2):
            engine.generate_batch(prompts, opts)
        engine.stats = type(engine.stats)()
    ran0 = dict(engine.decoder.counts) if engine.decoder is not None else {}
    steps0 = engine.runner.steps_run
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate_batch(prompts, opts)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = engine.stats
    return {"workload": "mixed", "requests": n_req, "prompt_tokens": sum(lens),
            "generated": sum(len(o) for o in outs), "seconds": dt,
            "total_tok_s": (sum(lens) + sum(len(o) for o in outs)) / dt,
            "decode_tok_s": sum(len(o) for o in outs) / dt, "steps": st.steps,
            "prefill_tokens": st.prefill_tokens, "decode_tokens": st.decode_tokens,
            "tokens_per_step": (st.prefill_tokens + st.decode_tokens) / max(st.steps, 1),
            "budget_use": (st.prefill_tokens + st.decode_tokens) / max(st.steps, 1) / (512 + n_req),
            # the host's own work per step against the step's whole time (the difference is spent
            # waiting for the device: a step is bound by the device while the former is the smaller)
            "host_ms_per_step": 1e3 * (st.step_seconds - st.wait_seconds) / max(st.steps, 1),
            "ms_per_step": 1e3 * dt / max(st.steps, 1), "preemptions": st.preemptions,
            # steps launched behind the step in flight, before its tokens were read
            "steps_launched_ahead": st.ahead_launched,
            # how the timed steps ran: replayed from a recording, recorded just then, or kernel by kernel
            "steps_run": {**{k: v - ran0.get(k, 0) for k, v in (engine.decoder.counts if engine.decoder else {}).items()},
                          "all": engine.runner.steps_run - steps0,
                          "recordings_kept": len(engine.decoder._slots) if engine.decoder else 0}}


def run_pressure(model, args) -> dict:
    import torch

    import infernum_b200 as ib

    n_req = args.requests or 32
    prompt_len = args.prompt_len or 2048
    new_tokens = args.new_tokens or 512
    vocab = model.spec.vocab_size
    rng = random.Random(args.seed)
    prompts = [[rng.randrange(vocab) for _ in range(prompt_len)] for _ in range(n_req)]
    per_req = -(-(prompt_len + new_tokens) // args.block_size)
    blocks = args.num_blocks or int(0.8 * n_req * per_req)  # deliberately too few
    opts = ib.GenerateOptions(max_new_tokens=new_tokens, ignore_eos=True)
    cfg = dict(max_batch_size=n_req, max_prefill_tokens=512, block_size=args.block_size,
               max_tokens_per_step=512 + n_req, max_model_len=prompt_len + new_tokens + 1)
    tight = ib.Engine(model, ib.BatchConfig(num_blocks=blocks, **cfg))
    if not args.no_warmup:
        # one untimed pass: the steps' shapes are recorded (the timed pass replays them)
        tight.run_until_done([tight.submit(p, opts) for p in prompts])
        tight.stats = type(tight.stats)()
        tight.scheduler.num_preemptions = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    handles = [tight.submit(p, opts) for p in prompts]
    tight.run_until_done(handles)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    outs = [h.tokens for h in handles]
    preemptions = tight.stats.preemptions
    preempted = [i for i, h in enumerate(handles) if h.seq.preemptions > 0]
    st = tight.stats
    del tight
    torch.cuda.empty_cache()
    # requests alone, with room: the yardstick (those that were preempted first)
    order = preempted + [i for i in range(n_req) if i not in preempted]
    checks = order if getattr(args, "solo_checks", None) is None else order[: args.solo_checks]
    solo = ib.Engine(model, ib.BatchConfig(num_blocks=per_req + 2, **dict(cfg, max_batch_size=1)))
    same, first_diff, gaps = 0, [], []
    for i in checks:
        want = solo.generate(prompts[i], opts)
        if want == outs[i]:
            same += 1
            continue
        k = next(k for k in range(len(want)) if outs[i][k] != want[k])
        first_diff.append(k)
        # how far apart the two tokens are by the engine's own logits at that step, as a
        # fraction of the largest: rounding can only turn a near-tie
        from ..engine.step import StepEntry

        rc = solo.cache.admit(("gap", i))
        seq, pos, logits = prompts[i] + want[:k], 0, None
        while pos < len(seq):
            n = min(512, solo.runner.max_rows, len(seq) - pos)
            logits = solo.runner.step([StepEntry(rc, seq[pos: pos + n], [n - 1] if pos + n == len(seq) else [])])
            pos += n
        row = logits[0].float()
        gaps.append(float((row[want[k]] - row[outs[i][k]]).abs() / row.abs().max()))
        solo.cache.release(rc)
    return {"workload": "pressure", "requests": n_req, "num_blocks": blocks,
            "blocks_for_all": n_req * per_req, "preemptions": preemptions,
            "requests_preempted": len(preempted), "prefill_tokens": st.prefill_tokens,
            "decode_tokens": st.decode_tokens, "steps": st.steps,
            "generated": sum(len(o) for o in outs), "seconds": dt,
            "total_tok_s": (st.prefill_tokens + st.decode_tokens) / dt,
            "decode_tok_s": sum(len(o) for o in outs) / dt, "solo_checked": len(checks),
            "identical_to_solo": same, "first_difference_at": first_diff,
            "logit_gap_at_first_difference": [round(g, 4) for g in gaps]}


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.gpus != 1:
        print("bench: this engine runs on one GPU (--gpus 1)", file=sys.stderr)
        return 2
    model = load(args)
    result = {"single": run_single, "mixed": run_mixed, "pressure": run_pressure}[args.workload](model, args)
    if args.json:
        print(json.dumps({k: (round(v, 3) if isinstance(v, float) else v) for k, v in result.items()}))
    elif args.workload == "single" and args.graph:
        print(f"{result['prefill_tokens']} tokens in {result['prefill_tokens'] / result['prefill_tok_s']:.4f}s = "
              f"{result['prefill_tok_s']:.1f} tok/s")
    elif args.workload == "single":
        print(f"{result['generated']} tokens in {result['seconds']:.2f}s = {result['decode_tok_s']:.1f} tok/s")
        print(f"prefill {result['prefill_tokens']} tokens = {result['prefill_tok_s']:.1f} tok/s")
    else:
        for k, v in result.items():
            print(f"{k}: {v:.3f}" if isinstance(v, float) else f"{k}: {v}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
