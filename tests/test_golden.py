"""The plain implementation against outputs of the reference's own CUDA
kernels (``tests/golden/reference_kernels.safetensors``, made once on a GPU by
``tests/golden/make_golden.py`` from the unchanged ``.cu`` files of
infernum-rs/infernum): each part alone, and a whole forward pass of a tiny
random model in which everything but the matrix products was computed by the
reference's kernels.  The golden values are float32; the plain implementation
runs in float64."""
import json
import os

import pytest
import torch

import plain_llama as pl
from helpers import TINY_A

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.safetensors")


@pytest.fixture(scope="module")
def golden():
    from safetensors import safe_open
    with safe_open(GOLDEN, framework="pt") as fh:
        tensors = {k: fh.get_tensor(k) for k in fh.keys()}
        meta = json.loads(fh.metadata()["meta"])
    return tensors, meta


def close(got, want, tol=2e-6):
    want = want.double()
    return float((got.double() - want).abs().max() / want.abs().max()) < tol


def test_rms_norm(golden):
    t, meta = golden
    assert close(pl.rms_norm(t["rmsnorm.x"].double(), t["rmsnorm.w"].double(), meta["rmsnorm.eps"]), t["rmsnorm.out"])
    total = t["add_rmsnorm.residual"].double() + t["add_rmsnorm.x"].double()
    assert close(total, t["add_rmsnorm.sum"])
    assert close(pl.rms_norm(total, t["add_rmsnorm.w"].double(), meta["add_rmsnorm.eps"]), t["add_rmsnorm.out"])


def test_rope(golden):
    t, meta = golden
    x = t["rope.x"].double()
    positions = torch.arange(x.shape[0]) + meta["rope.offset"]
    freqs = pl.rope_frequencies(x.shape[2], meta["rope.theta"], None)
    assert close(pl.rope(x, positions, freqs), t["rope.out"])
    assert not close(pl.rope(x, positions + 1, freqs), t["rope.out"], 1e-2)


def test_attention(golden):
    t, meta = golden
    q, k, v = t["attention.q"].double(), t["attention.k"].double(), t["attention.v"].double()
    offset = meta["attention.offset"]
    assert offset + q.shape[0] == k.shape[0]
    # the plain function takes whole sequences: queries of the rows before the offset do not matter
    q_all = torch.cat([torch.zeros(offset, *q.shape[1:], dtype=q.dtype), q])
    assert close(pl.attention(q_all, k, v)[offset:], t["attention.out"])
    assert close(pl.attention(q_all, k, v, window=7)[offset:], t["attention.out_window7"])
    assert not close(t["attention.out"], t["attention.out_window7"], 1e-2)


def test_silu_mul(golden):
    t, _ = golden
    gate, up = t["silu_mul.gate"].double(), t["silu_mul.up"].double()
    n = gate.shape[1]
    eye, zero = torch.eye(n, dtype=torch.float64), torch.zeros(n, n, dtype=torch.float64)
    # the plain function is the whole feed-forward: with these matrices it reduces to silu(gate) * up
    got = pl.swiglu(torch.cat([gate, up], dim=1), torch.cat([eye, zero], dim=1), torch.cat([zero, eye], dim=1), eye)
    assert close(got, t["silu_mul.out"])


def test_embedding(golden):
    t, _ = golden
    assert torch.equal(pl.embedding(t["embedding.table"], t["embedding.ids"].tolist()), t["embedding.out"])


def test_whole_tiny_model(golden):
    """Logits of Tiny A over 21 tokens: the reference's kernels strung together in the
    order of its graph builder against ``plain_llama.forward``."""
    from infernum_b200.weights.random_init import model_specs_for, random_tensors
    t, meta = golden
    assert meta["model.config"] == "TINY_A"
    _, _, specs = model_specs_for(TINY_A)
    weights = random_tensors(specs, meta["model.seed"], "cpu", torch.float32)
    logits = pl.forward(pl.read_config(TINY_A), weights, meta["model.tokens"])
    assert logits.shape == t["model.logits"].shape
    assert close(logits, t["model.logits"], 1e-5)
