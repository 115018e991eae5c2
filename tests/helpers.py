"""Shared by the tests: the two tiny configurations, model folders in a
temporary place, traces, and the comparison rule."""

from __future__ import annotations

import io
import json
import os
import random
import subprocess
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

import plain_llama

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two configurations that differ in every size and option.
TINY_A = {
    "model_type": "llama", "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 176, "vocab_size": 256,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 128,
}
TINY_B = {
    "model_type": "llama", "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256, "vocab_size": 320,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256,
}
# A third one with sizes that are no power of two anywhere and a head size of 48.
TINY_C = {
    "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 120,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48,
    "intermediate_size": 200, "vocab_size": 333, "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "max_position_embeddings": 512,
}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
PAGE_SIZES = {"A": 4, "B": 8, "C": 16}

# Relative to the largest reference logit of the compared block.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def make_model_folder(folder: str, config: dict, seed: int, sharpen: float = 0.0) -> str:
    """Random model through the package's writer.  ``sharpen`` > 0 scales the
    query and key projections so that attention is peaked and a single wrong
    key shows in the logits."""
    from infernum_b200.weights.random_init import write_random_model

    write_random_model(folder, config, seed)
    if sharpen:
        from safetensors.torch import load_file, save_file

        path = os.path.join(folder, "model.safetensors")
        tensors = load_file(path)
        for name in list(tensors):
            if name.endswith(("q_proj.weight", "k_proj.weight")):
                tensors[name] = (tensors[name].float() * sharpen).to(torch.bfloat16)
            if name.endswith(("v_proj.weight", "o_proj.weight")):
                tensors[name] = (tensors[name].float() * 4.0).to(torch.bfloat16)
        save_file(tensors, path, metadata={"format": "pt"})
    return folder


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


class Plain:
    """The plain implementation over a model folder, logits cached by sequence."""

    def __init__(self, folder: Optional[str], config: Optional[dict] = None,
                 weights: Optional[Dict[str, torch.Tensor]] = None):
        """From a model folder, or from a config.json dict and CPU tensors by
        checkpoint name."""
        self.cfg = plain_llama.read_config(folder if folder is not None else config)
        self.weights = plain_llama.read_weights(folder) if folder is not None else weights
        self._cache: Dict[tuple, torch.Tensor] = {}

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._cache:
            self._cache[key] = plain_llama.forward(self.cfg, self.weights, list(tokens))
        return self._cache[key]


# --------------------------------------------------------------------------
# traces
# --------------------------------------------------------------------------
def run_trace_inprocess(model_dir: str, dtype: str, steps: List[dict], out_dir: str,
                        max_tokens: int, page_size: int) -> Dict[int, np.ndarray]:
    from infernum_b200.cli.trace_run import main

    stdin = io.StringIO("".join(json.dumps(s) + "\n" for s in steps))
    stdout = io.StringIO()
    rc = main(["--model", model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens",
               str(max_tokens), "--page-size", str(page_size)], stdin=stdin, stdout=stdout)
    assert rc == 0
    done = [l for l in stdout.getvalue().splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps]
    return read_outputs(out_dir, steps, model_dir)


def run_trace_subprocess(model_dir: str, dtype: str, steps: List[dict], out_dir: str,
                         max_tokens: int, env: Optional[dict] = None) -> Dict[int, np.ndarray]:
    proc = subprocess.run(
        [os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out",
         out_dir, "--max-tokens", str(max_tokens)],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
        env=env, timeout=900)
    assert proc.returncode == 0, proc.stderr[-4000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps]
    return read_outputs(out_dir, steps, model_dir)


def read_outputs(out_dir: str, steps: List[dict], model_dir: str) -> Dict[int, np.ndarray]:
    vocab = json.load(open(os.path.join(model_dir, "config.json")))["vocab_size"]
    out = {}
    for s in steps:
        wanted = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if wanted:
            arr = np.fromfile(path, dtype="<f4")
            assert arr.size == wanted * vocab, (s["step"], arr.size, wanted, vocab)
            out[s["step"]] = arr.reshape(wanted, vocab)
        else:
            assert not os.path.exists(path)
    return out


def compare_trace(steps: List[dict], outputs: Dict[int, np.ndarray],
                  sequences: Dict[str, List[int]], plain: Plain, tol: float) -> float:
    """Every wanted row against the plain implementation's logits at the same
    (request, position).  Returns the worst relative error; asserts on the
    first row beyond ``tol`` and says where it is."""
    fed = {rid: 0 for rid in sequences}
    worst = 0.0
    for s in steps:
        row = 0
        for e in s["entries"]:
            rid, n = e["id"], len(e["tokens"])
            assert e["tokens"] == sequences[rid][fed[rid]: fed[rid] + n], "trace feeds wrong tokens"
            ref_all = plain.logits(sequences[rid])
            for w in e.get("want", []):
                pos = fed[rid] + w
                ref = ref_all[pos].numpy()
                got = outputs[s["step"]][row]
                err = float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-6))
                worst = max(worst, err)
                assert np.isfinite(got).all(), f"step {s['step']} request {rid} pos {pos}: not finite"
                assert err <= tol, (f"step {s['step']} request {rid} position {pos} "
                                    f"(place {w} of a portion of {n} starting at {fed[rid]}): "
                                    f"relative error {err:.3e} > {tol:.1e}")
                row += 1
            fed[rid] += n
        for rid in s.get("end", []):
            fed[rid] = 0
    return worst


def trace_whole(rid: str, seq: List[int], step0: int = 0) -> List[dict]:
    return [{"step": step0, "entries": [{"id": rid, "tokens": seq, "want": list(range(len(seq)))}],
             "end": [rid]}]


def trace_tail(rid: str, seq: List[int], tail: int = 32, step0: int = 0) -> List[dict]:
    """Most of it in one step, the last ``tail`` tokens one by one."""
    head = max(1, len(seq) - tail)
    steps = [{"step": step0, "entries": [{"id": rid, "tokens": seq[:head], "want": [head - 1]}],
              "end": []}]
    for i in range(head, len(seq)):
        steps.append({"step": step0 + len(steps),
                      "entries": [{"id": rid, "tokens": [seq[i]], "want": [0]}], "end": []})
    steps[-1]["end"] = [rid]
    return steps


def trace_portions(rid: str, seq: List[int], sizes: Sequence[int], step0: int = 0) -> List[dict]:
    """Portions of changing size (cycled) until the sequence is consumed."""
    steps, pos, i = [], 0, 0
    while pos < len(seq):
        n = min(sizes[i % len(sizes)], len(seq) - pos)
        steps.append({"step": step0 + len(steps),
                      "entries": [{"id": rid, "tokens": seq[pos: pos + n],
                                   "want": sorted({0, n - 1})}], "end": []})
        pos += n
        i += 1
    steps[-1]["end"] = [rid]
    return steps


def trace_mixed(sequences: Dict[str, List[int]], max_live: int, seed: int,
                decode_tail: int = 12) -> List[dict]:
    """Up to ``max_live`` requests at a time: portions of prompts beside single
    decoded tokens of others; a request may sit out a step; a finished one is
    replaced by the next, so its pages are used again."""
    rng = random.Random(seed)
    waiting = list(sequences)
    live: Dict[str, int] = {}
    steps: List[dict] = []
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            seq, pos = sequences[rid], live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            left = len(seq) - pos
            n = 1 if left <= decode_tail else min(left - decode_tail, rng.choice([2, 3, 5, 7, 11, 19]))
            want = [n - 1] if n == 1 or rng.random() < 0.7 else []
            entries.append({"id": rid, "tokens": seq[pos: pos + n], "want": want})
            live[rid] = pos + n
            if live[rid] == len(seq):
                end.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def peak_tokens(steps: List[dict]) -> int:
    """Most tokens live requests hold at any time, each rounded up to 64."""
    held: Dict[str, int] = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((v + 63) // 64 * 64 for v in held.values()))
        for rid in s.get("end", []):
            held.pop(rid, None)
    return peak


# --------------------------------------------------------------------------
# generated tokens
# --------------------------------------------------------------------------
TIE = {"float32": 1e-4, "bfloat16": 5e-2}


def assert_same_up_to_ties(folder_or_plain, prompt: Sequence[int], got: Sequence[int], want: Sequence[int],
                           dtype: str, sampling=None) -> int:
    """Two token lists for one request must be equal, up to the first step that
    the plain implementation calls a near-tie: two runs that went through
    different kernels or batches may round such a step differently, and nothing
    after it can be compared.  Everything before it is.

    Greedy: at the first difference the two tokens' plain logits differ by less
    than ``TIE[dtype]`` of the largest logit.  Sampled (``sampling`` has
    temperature, top_p, seed, repetition_penalty and its window): the step's
    uniform number lies within ``TIE[dtype]`` of the interval that the plain
    distribution gives to the token that was got.  Returns the number of
    tokens that were compared and equal."""
    got, want = list(got), list(want)
    if got == want:
        return len(got)
    i = next((k for k in range(min(len(got), len(want))) if got[k] != want[k]), None)
    assert i is not None, f"lengths differ: {len(got)} against {len(want)} tokens"
    plain = folder_or_plain if isinstance(folder_or_plain, Plain) else Plain(folder_or_plain)
    seq = list(prompt) + want[:i]
    logits = plain.logits(seq)[-1]
    limit = TIE[dtype]
    if sampling is None:
        gap = float((logits[want[i]] - logits[got[i]]).abs() / logits.abs().max())
        assert gap < limit, (f"token {i}: {got[i]} against {want[i]}, whose plain logits differ by {gap:.4f} "
                             f"of the largest: no near-tie")
        return i
    w = sampling.repetition_penalty_window
    recent = seq[len(seq) - w:] if w else []
    probs = plain_llama.sample_probabilities(logits, sampling.temperature, sampling.top_p,
                                             sampling.repetition_penalty, recent)
    u = plain_llama.uniform_number(sampling.seed, i)
    cdf = torch.cumsum(probs, dim=0)
    hi = float(cdf[got[i]])
    lo = hi - float(probs[got[i]])
    away = max(lo - u, u - hi, 0.0)
    assert away < limit, (f"sampled token {i}: {got[i]} against {want[i]}; u = {u:.4f} lies {away:.4f} away from "
                          f"the plain interval [{lo:.4f}, {hi:.4f}) of the token that was got")
    return i
