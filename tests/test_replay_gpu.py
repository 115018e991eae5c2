"""Trace replay on the GPU against the plain implementation, in 32-bit and in
bfloat16: each request alone and whole; most of it in one step and the last 32
tokens one by one; in portions of changing size, down to two tokens; and
mixed, up to four live requests with so few pages that they are used again."""
import os

import numpy as np
import pytest

from helpers import (CONFIGS, PAGE_SIZES, TOL, Plain, compare_trace, make_model_folder,
                     peak_tokens, random_tokens, run_trace_inprocess, run_trace_subprocess,
                     trace_mixed, trace_portions, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [21, 33, 49, 100, 1, 2], "B": [25, 40, 64, 124, 1, 9], "C": [77, 130, 18, 200, 3, 64]}
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        folder = make_model_folder(str(tmp_path_factory.mktemp(f"model{name}")), cfg, seed=20 + len(out))
        sharp = make_model_folder(str(tmp_path_factory.mktemp(f"sharp{name}")), cfg, seed=40 + len(out),
                                  sharpen=6.0)
        out[name] = (folder, Plain(folder))
        out[name + "sharp"] = (sharp, Plain(sharp))
    return out


def sequences(name):
    key = name.replace("sharp", "")
    vocab = CONFIGS[key]["vocab_size"]
    return {f"r{i}": random_tokens(n, vocab, 100 * i + n) for i, n in enumerate(LENGTHS[key])}


def replay(models, name, dtype, steps, tmp_path, max_tokens=None):
    folder, plain = models[name]
    key = name.replace("sharp", "")
    outputs = run_trace_inprocess(folder, dtype, steps, str(tmp_path / "out"),
                                  max_tokens or peak_tokens(steps), PAGE_SIZES[key])
    return outputs, plain


NAMES = ["A", "B", "C", "Asharp", "Bsharp"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(models, name, dtype, tmp_path):
    seqs = sequences(name)
    steps = []
    for rid, seq in seqs.items():
        steps += trace_whole(rid, seq, step0=len(steps))
    outputs, plain = replay(models, name, dtype, steps, tmp_path)
    compare_trace(steps, outputs, seqs, plain, TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_most_in_one_step_then_the_last_32_one_by_one(models, name, dtype, tmp_path):
    seqs = {k: v for k, v in sequences(name).items() if len(v) > 3}
    steps = []
    for rid, seq in seqs.items():
        steps += trace_tail(rid, seq, 32, step0=len(steps))
    outputs, plain = replay(models, name, dtype, steps, tmp_path)
    compare_trace(steps, outputs, seqs, plain, TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_changing_size(models, name, dtype, tmp_path):
    seqs = {k: v for k, v in sequences(name).items() if len(v) > 3}
    steps = []
    for i, (rid, seq) in enumerate(seqs.items()):
        sizes = [[7, 2, 5, 3, 11, 2], [2, 2, 13, 4, 2, 9], [5, 17, 2, 3], [2]][i % 4]
        steps += trace_portions(rid, seq, sizes, step0=len(steps))
    outputs, plain = replay(models, name, dtype, steps, tmp_path)
    compare_trace(steps, outputs, seqs, plain, TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_with_pages_used_again(models, name, dtype, tmp_path):
    seqs = sequences(name)
    steps = trace_mixed(seqs, max_live=4, seed=7)
    assert max(len(s["entries"]) for s in steps) >= 3
    assert any(len(e["tokens"]) > 1 for s in steps if len(s["entries"]) > 1 for e in s["entries"])
    peak = peak_tokens(steps)
    total = sum((len(v) + 63) // 64 * 64 for v in seqs.values())
    assert peak < total  # the pool is smaller than all requests together: pages come back
    outputs, plain = replay(models, name, dtype, steps, tmp_path, max_tokens=peak)
    compare_trace(steps, outputs, seqs, plain, TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(models, dtype, tmp_path):
    seqs = {"long": random_tokens(250, CONFIGS["B"]["vocab_size"], 9)}
    steps = trace_tail("long", seqs["long"], tail=244)
    outputs, plain = replay(models, "B", dtype, steps, tmp_path)
    compare_trace(steps, outputs, seqs, plain, TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_does_not_change_logits_beyond_rounding(models, dtype, tmp_path):
    """The same positions through three ways of cutting agree with each other
    far more closely than bfloat16 agrees with the plain implementation."""
    seq = sequences("B")["r3"]
    seqs = {"r3": seq}
    runs = []
    for i, steps in enumerate([trace_whole("r3", seq), trace_portions("r3", seq, [7, 2, 5, 3, 11, 2]),
                               trace_tail("r3", seq, 32)]):
        folder, _ = models["B"]
        out = run_trace_inprocess(folder, dtype, steps, str(tmp_path / f"o{i}"), 128, 8)
        rows, pos = {}, 0
        for s in steps:
            r = 0
            for e in s["entries"]:
                for w in e["want"]:
                    rows[pos + w] = out[s["step"]][r]
                    r += 1
                pos += len(e["tokens"])
        runs.append(rows)
    scale = max(np.abs(v).max() for v in runs[0].values())
    tol = 1e-5 if dtype == "float32" else 2e-2
    for other in runs[1:]:
        for pos, row in other.items():
            assert np.abs(row - runs[0][pos]).max() / scale <= tol, f"position {pos}"


def test_the_program_itself_in_a_subprocess(models, tmp_path):
    folder, plain = models["A"]
    seqs = {k: v for k, v in sequences("A").items() if len(v) > 3}
    steps = trace_mixed(seqs, max_live=3, seed=3)
    outputs = run_trace_subprocess(folder, "float32", steps, str(tmp_path / "out"), peak_tokens(steps))
    compare_trace(steps, outputs, seqs, plain, TOL["float32"])
    outputs = run_trace_subprocess(folder, "bfloat16", steps, str(tmp_path / "out2"), peak_tokens(steps))
    compare_trace(steps, outputs, seqs, plain, TOL["bfloat16"])
