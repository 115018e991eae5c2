#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decoded tokens per second at the
Llama-3.1-8B layer sizes with random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W]

A "step" is one decode step of the whole batch.  The default run: batch 8,
prompts of 1,024 tokens, K timed decode steps after W untimed ones.  One JSON
line is printed:

  value      decoded tokens per second, timed on the device with CUDA events
             around K steps whose inputs stay on the device
  e2e        the same through the Python entry point (``Engine``): host tokens
             in (pinned memory, copied every step) and host tokens out
  prefill    one step over a 2,048-token prompt: tokens/s, time, and the
             fraction of the measured bf16 matmul peak its flops reach
  roofline   bytes a decode step must read (every weight once, the cache of
             the live requests) / its time, against the measured copy bandwidth
  points     decode tokens/s at batch 1 and at batch 64 (1,024-token prompts), and
             at batch 8 near the end of an 8,192-token context; and two runs
             through the scheduler at other layer sizes, each with a model of its
             own made after the headline runs: the Llama-3.2-1B sizes under a
             mixed workload (64 requests, prompts of 16 to 4,096 tokens fed 512
             at a time beside decoding requests, temperature 0.8), and the
             Llama-2-13B sizes with a page pool of 0.8 of the need, so that
             requests are preempted and recomputed (``pressure_13b_*``; some of
             them, the preempted ones first, are run again alone and compared)

Weights (15 GB) and cache are far larger than the 126 MB L2, so every timed
step streams its inputs from HBM; no L2 flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_8B = {
    "model_type": "llama", "num_hidden_layers": 32, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192,
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            p = json.load(fh)
        p["source"] = "measured"
        return p
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0: float, t1: float):
        rows = [l for t, l in self.samples if t0 <= t <= t1] or [l for _, l in self.samples[-3:]]
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in rows:
            parts = [x.strip() for x in l.split(",")]
            try:
                mhz.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def decode_bytes(model, cache, live_tokens: int) -> int:
    """Bytes one decode step has to read: every weight it uses once, and the
    keys and values of the live requests."""
    return model.step_weight_bytes() + cache.bytes_per_token() * live_tokens


def prefill_flops(cfg: dict, T: int, layers: int) -> float:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2.0 * T * H * ((nh + 2 * nkv) * hd) + 2.0 * T * (nh * hd) * H + 2.0 * T * H * 2 * I + 2.0 * T * I * H
    attn = 2.0 * 2.0 * nh * hd * T * (T + 1) / 2.0  # causal: QK^T and PV
    return layers * (linear + attn) + 2.0 * 1 * H * V


def make_requests(runner, cache, batch, prompt_len, vocab, seed, chunk=2048):
    """Admits ``batch`` requests and runs their prompts through the step
    function in portions of at most ``chunk`` tokens.  Returns the caches and
    the first token selected for each."""
    import torch

    from infernum_b200.engine.step import StepEntry
    from infernum_b200.ops import core

    g = torch.Generator().manual_seed(seed)
    caches, first = [], []
    for b in range(batch):
        rc = cache.admit(("bench", seed, b))
        prompt = torch.randint(0, vocab, (prompt_len,), generator=g).tolist()
        pos, logits = 0, None
        while pos < prompt_len:
            n = min(chunk, prompt_len - pos)
            logits = runner.step([StepEntry(rc, prompt[pos: pos + n], [n - 1] if pos + n == prompt_len else [])])
            pos += n
        out = torch.empty(1, dtype=torch.int32, device=logits.device)
        core.argmax(logits, out)
        caches.append(rc)
        first.append(int(out.item()))
    return caches, first


def time_decode(model, batch, prompt_len, steps, warmup, page_size, seed, clocks=None, graph=True):
    """Device-timed decode: K steps of a DecodeRunner that feeds itself."""
    import torch

    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.decode import DecodeRunner
    from infernum_b200.engine.step import ModelRunner
    from infernum_b200.ops import core

    total = prompt_len + steps + warmup + 8
    pages = batch * (-(-total // page_size)) + 8
    cache = CacheManager(model.cache_needs(), page_size=page_size, num_pages=pages, max_requests=batch,
                         dtype=model.rt.dtype, device=model.rt.device)
    runner = ModelRunner(model, cache, max_rows=4096, max_entries=max(batch, 1))
    caches, first = make_requests(runner, cache, batch, prompt_len, model.spec.vocab_size, seed)
    session = DecodeRunner(runner, total + 8, use_graph=graph)
    session.pin(caches, first, steps + max(warmup, 3) + 2)
    for _ in range(max(warmup, 3)):
        session.step_pinned()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = core.LAUNCHES
    t0 = time.time()
    start.record()
    for _ in range(steps):
        session.step_pinned()
    end.record()
    torch.cuda.synchronize()
    t1 = time.time()
    runner.check_errors()
    ms = start.elapsed_time(end) / steps
    live = sum(rc.num_tokens for rc in caches) - batch * steps // 2  # mean over the timed steps
    result = {
        "ms_per_step": ms, "tokens_per_s": batch * 1000.0 / ms,
        "bytes_per_step": decode_bytes(model, cache, live),
        "launches_per_step": session.last.launches_per_step,
        "graph": session.last.graph is not None,
        "clocks": clocks.summary(t0, t1) if clocks else None,
    }
    for rc in caches:
        cache.release(rc)
    del session, runner, cache
    torch.cuda.empty_cache()
    return result


def time_e2e(model, batch, prompt_len, steps, warmup, page_size, seed, launch_ahead=True):
    """The same through ``Engine``: requests are submitted as host token lists,
    every step copies its inputs from pinned memory and reads the selected
    tokens back.  With ``launch_ahead`` (the engine's default) a decode step is
    launched behind the one in flight and takes that one's tokens on the device;
    its positions, lengths and slots still come from the host every step.
    Without it every step is launched after the one before was read and gets
    its tokens from the host too."""
    import torch

    import infernum_b200 as ib

    total = prompt_len + steps + warmup + 8
    pages = batch * (-(-total // page_size)) + 8
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=batch, max_prefill_tokens=2048,
                                             block_size=page_size, num_blocks=pages,
                                             max_tokens_per_step=2048, max_model_len=total + 8,
                                             launch_ahead=launch_ahead))
    g = torch.Generator().manual_seed(seed)
    opts = ib.GenerateOptions(max_new_tokens=steps + warmup + 6, ignore_eos=True)
    handles = [engine.submit(torch.randint(0, model.spec.vocab_size, (prompt_len,), generator=g).tolist(), opts)
               for _ in range(batch)]
    while any(len(h.seq.generated_ids) < 1 for h in handles):
        engine.step()  # prompts
    for _ in range(max(warmup, 3)):
        engine.step()
    torch.cuda.synchronize()
    before = sum(len(h.seq.generated_ids) for h in handles)
    h2d0, d2h0 = engine.h2d_bytes, engine.d2h_bytes
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    made = sum(len(h.seq.generated_ids) for h in handles) - before
    for h in handles:
        engine.cancel(h)
    engine.step()
    out = {"value": made / dt, "unit": "tokens/s", "ms_per_step": dt * 1000 / steps,
           "h2d_bytes_per_step": (engine.h2d_bytes - h2d0) / steps,
           "d2h_bytes_per_step": (engine.d2h_bytes - d2h0) / steps}
    del engine
    torch.cuda.empty_cache()
    return out


def time_prefill(model, cfg, layers, T, page_size, peaks, reps=3, recorded=False):
    """One step over a whole prompt of ``T`` tokens, timed on the device.
    ``recorded``: the way ``Engine`` runs a prompt that comes alone - replayed from
    a recording made for the bucket of its length - with the host's own time for
    the step beside it (a step is bound by the device while that is the smaller)."""
    import torch

    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.decode import DecodeRunner
    from infernum_b200.engine.step import ModelRunner, StepEntry

    cache = CacheManager(model.cache_needs(), page_size=page_size, num_pages=-(-T // page_size) + 2,
                         max_requests=1, dtype=model.rt.dtype, device=model.rt.device)
    runner = ModelRunner(model, cache, max_rows=T, max_entries=1)
    session = DecodeRunner(runner, T + 8) if recorded else None
    g = torch.Generator().manual_seed(5)
    times, host = [], []
    for i in range(reps + (3 if recorded else 2)):
        prompt = torch.randint(0, model.spec.vocab_size, (T,), generator=g).tolist()
        rc = cache.admit(("prefill", i))
        cache.extend(rc, T)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        if recorded:
            slot = session.prepare([], 0, portions=[(rc, T, True)])
            session.launch(slot, [], [], None, portions=[(rc, prompt, True)])
        else:
            runner.step([StepEntry(rc, prompt, [T - 1])])
        end.record()
        t1 = time.perf_counter()
        torch.cuda.synchronize()
        if recorded:
            session.read_result(0, [0])
        if i >= (3 if recorded else 2):
            times.append(start.elapsed_time(end))
            host.append((t1 - t0) * 1e3)
        cache.release(rc)
    runner.check_errors()
    ms = sorted(times)[len(times) // 2]
    flops = prefill_flops(cfg, T, layers)
    peak = peaks["bf16_tflops_sustained"]
    del runner, cache
    torch.cuda.empty_cache()
    return {"value": T * 1000.0 / ms, "tokens": T, "ms": ms, "host_ms": sorted(host)[len(host) // 2],
            "frac": flops / (ms * 1e-3) / (peak * 1e12), "tflops": flops / (ms * 1e-3) / 1e12,
            "peak_tflops": peak,
            # the same against the burst rate of the library product (a kernel timed in isolation)
            "frac_of_burst": flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)}


def scheduler_workloads(seed: int) -> dict:
    """The mixed workload at the 1B layer sizes and the page-pressure workload at
    the 13B layer sizes, through ``Engine`` (``infernum_b200.cli.bench``), as
    flat entries for ``points``."""
    import gc
    from types import SimpleNamespace

    import torch

    from infernum_b200.cli import bench as cli

    out = {}
    base = dict(dtype="bf16", layers=None, seed=seed, block_size=16, requests=None, prompt_len=None,
                new_tokens=None, num_blocks=None, no_warmup=False, n_gen=128)
    args = SimpleNamespace(model="1b", workload="mixed", **base)
    model = cli.load(args)
    r = cli.run_mixed(model, args)
    out.update({"mixed_1b_tok_s": round(r["total_tok_s"], 1), "mixed_1b_decode_tok_s": round(r["decode_tok_s"], 1),
                "mixed_1b_prefill_tokens": r["prefill_tokens"], "mixed_1b_decode_tokens": r["decode_tokens"],
                "mixed_1b_steps": r["steps"], "mixed_1b_budget_use": round(r["budget_use"], 3),
                "mixed_1b_ms_per_step": round(r["ms_per_step"], 3),
                "mixed_1b_host_ms_per_step": round(r["host_ms_per_step"], 3),
                "mixed_1b_steps_replayed": r["steps_run"].get("replayed", 0),
                "mixed_1b_steps_launched_ahead": r.get("steps_launched_ahead", 0),
                "mixed_1b_preemptions": r["preemptions"]})
    del model
    gc.collect()
    torch.cuda.empty_cache()
    args = SimpleNamespace(model="13b", workload="pressure", solo_checks=4, **base)
    model = cli.load(args)
    r = cli.run_pressure(model, args)
    out.update({"pressure_13b_tok_s": round(r["total_tok_s"], 1), "pressure_13b_decode_tok_s": round(r["decode_tok_s"], 1),
                "pressure_13b_layers": len(model.layers), "pressure_13b_num_blocks": r["num_blocks"],
                "pressure_13b_blocks_for_all": r["blocks_for_all"], "pressure_13b_preemptions": r["preemptions"],
                "pressure_13b_requests_preempted": r["requests_preempted"],
                "pressure_13b_solo_checked": r["solo_checked"],
                "pressure_13b_identical_to_solo": r["identical_to_solo"],
                "pressure_13b_first_difference_at": ",".join(str(i) for i in r["first_difference_at"]),
                # (bfloat16, random weights: a differing token must be a near-tie by the logits)
                "pressure_13b_largest_gap_at_difference": max(r["logit_gap_at_first_difference"] + [0.0])})
    del model
    gc.collect()
    torch.cuda.empty_cache()
    # the same in true 32-bit, where a preempted request must reproduce its tokens exactly
    # (four layers and eight requests: the 32-bit products run on the FMA units)
    args = SimpleNamespace(model="13b", workload="pressure", solo_checks=4,
                           **dict(base, dtype="f32", layers=4, requests=8, prompt_len=1024, new_tokens=256))
    model = cli.load(args)
    r = cli.run_pressure(model, args)
    out.update({"pressure_13b_f32_layers": 4, "pressure_13b_f32_requests": 8, "pressure_13b_f32_prompt_len": 1024,
                "pressure_13b_f32_preemptions": r["preemptions"],
                "pressure_13b_f32_solo_checked": r["solo_checked"],
                "pressure_13b_f32_identical_to_solo": r["identical_to_solo"]})
    del model
    gc.collect()
    torch.cuda.empty_cache()
    return out


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--skip-extras", action="store_true", help="only the headline decode run")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one part only and print its numbers (for profiling)")
    ap.add_argument("--no-cuda-graph", action="store_true", help="launch decode steps kernel by kernel")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "infernum-rs/infernum is a Rust workspace; neither cargo nor rustc is "
                          "installed here and it has no Python package to install offline"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)

    import torch

    import infernum_b200 as ib
    from infernum_b200.csrc.build import loaded_libraries

    peaks = load_peaks()
    cfg = dict(LLAMA_8B)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    torch.cuda.set_device(0)
    model = ib.random_model(cfg, seed=args.seed, dtype="bfloat16", device="cuda:0",
                            options={"sm_count": torch.cuda.get_device_properties(0).multi_processor_count})
    if args.only == "decode":
        r = time_decode(model, args.batch, args.prompt_len, args.steps, warmup, args.page_size, args.seed,
                        graph=not args.no_cuda_graph)
        print(json.dumps({"only": "decode", "batch": args.batch, **r}))
        return 0
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", **time_prefill(model, cfg, layers, 2048, args.page_size, peaks)}))
        return 0
    clocks = ClockSampler(0)
    clocks.start()
    try:
        # The prompt step is bound by arithmetic and so by the SM clock, which sags under the
        # power cap once the decode runs have heated the part (decode is bound by HBM): it is
        # timed here, on the cool part, and again after the decode runs; the line carries the
        # later, slower figure and names the earlier one beside it.
        cool = None if args.skip_extras else time_prefill(model, cfg, layers, 2048, args.page_size, peaks)
        main_run = time_decode(model, args.batch, args.prompt_len, args.steps, warmup, args.page_size,
                               args.seed, clocks)
        e2e = time_e2e(model, args.batch, args.prompt_len, args.steps, warmup, args.page_size, args.seed + 1)
        e2e["tokens"] = "fed on the device to a step launched ahead; positions, lengths and slots from the host"
        if not args.skip_extras:
            fed = time_e2e(model, args.batch, args.prompt_len, min(args.steps, 64), warmup, args.page_size,
                           args.seed + 1, launch_ahead=False)
            e2e["value_host_fed"] = round(fed["value"], 2)  # every step launched after the one before was read
            e2e["h2d_bytes_per_step_host_fed"] = fed["h2d_bytes_per_step"]
        points = {}
        if not args.skip_extras:
            for b in (1, 64):
                r = time_decode(model, b, args.prompt_len, min(args.steps, 64), warmup, args.page_size,
                                args.seed + 2 + b)
                points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
                points[f"decode_b{b}_hbm_frac"] = round(
                    r["bytes_per_step"] / (r["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
            # the same batch of 8 near the end of the 8,192-token context the configuration names
            r = time_decode(model, 8, 8192 - 128, 32, warmup, args.page_size, args.seed + 9)
            points["decode_b8_ctx8k"] = round(r["tokens_per_s"], 1)
            points["decode_b8_ctx8k_hbm_frac"] = round(
                r["bytes_per_step"] / (r["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
        if not args.skip_extras:
            # short prompts, the way the engine runs a prompt that comes alone: device time, the
            # host's own time for the step, and the fraction of the sustained bf16 rate
            for T in (256, 512):
                r = time_prefill(model, cfg, layers, T, args.page_size, peaks, recorded=True)
                points[f"prefill_{T}_ms"] = round(r["ms"], 3)
                points[f"prefill_{T}_host_ms"] = round(r["host_ms"], 3)
                points[f"prefill_{T}_frac"] = round(r["frac"], 4)
        prefill = None
        if cool is not None:
            prefill = time_prefill(model, cfg, layers, 2048, args.page_size, peaks)
            prefill.update({"when": "after the decode runs", "ms_cool": cool["ms"], "frac_cool": cool["frac"],
                            "value_cool": cool["value"]})
        libraries = [os.path.basename(p) for p in loaded_libraries()]
        if not args.skip_extras and not args.layers:
            del model
            import gc

            gc.collect()
            torch.cuda.empty_cache()
            points.update(scheduler_workloads(args.seed))
    finally:
        clocks.stop()

    achieved = main_run["bytes_per_step"] / (main_run["ms_per_step"] * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s (Llama-3.1-8B layer sizes, random bf16 weights)",
        "value": round(main_run["tokens_per_s"], 2),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0, 0.02), seeded uniform token ids",
        "config": {
            "model": "llama-3.1-8b-shape", "layers": layers, "layers_full": full_layers,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": args.batch, "seq_len": args.prompt_len, "context_len": 8192,
            "page_size": args.page_size, "parallelism": "single-gpu",
            "l2": "inputs larger than L2 (15 GB of weights per step)",
            "cuda_graph": bool(main_run["graph"]),
        },
        "clocks": main_run["clocks"],
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(main_run["launches_per_step"]) * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                     "peaks": peaks["source"]},
        "points": points,
        "kernel_libraries": libraries,
    }
    if prefill is not None:
        line["prefill"] = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in prefill.items()}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
