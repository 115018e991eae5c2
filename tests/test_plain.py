"""The plain implementation checked against itself and against hand-made
cases (no GPU): it is the yardstick of every GPU test, so its own parts are
pinned here."""
import math

import pytest
import torch

import plain_llama as pl
from helpers import TINY_A, TINY_B, make_model_folder, random_tokens


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    inv = 1 / math.sqrt((9 + 16) / 2 + 1e-5)
    assert torch.allclose(pl.rms_norm(x, w, 1e-5), torch.tensor([[3 * inv * 2, 4 * inv * 0.5]], dtype=torch.float64))


def test_rope_pairs_and_position_zero():
    x = torch.arange(8, dtype=torch.float64).view(1, 1, 8)
    f = pl.rope_frequencies(8, 10000.0, None)
    assert torch.equal(pl.rope(x, torch.tensor([0]), f), x)
    y = pl.rope(x, torch.tensor([3]), f)
    for j in range(4):
        a = 3 * float(f[j])
        assert y[0, 0, j].item() == pytest.approx(x[0, 0, j] * math.cos(a) - x[0, 0, j + 4] * math.sin(a), abs=1e-6)
        assert y[0, 0, j + 4].item() == pytest.approx(x[0, 0, j] * math.sin(a) + x[0, 0, j + 4] * math.cos(a), abs=1e-6)
    # a rotation keeps the norm, and q.k depends on the distance only
    q = torch.randn(1, 1, 8, dtype=torch.float64)
    k = torch.randn(1, 1, 8, dtype=torch.float64)
    d1 = (pl.rope(q, torch.tensor([7]), f) * pl.rope(k, torch.tensor([2]), f)).sum()
    d2 = (pl.rope(q, torch.tensor([25]), f) * pl.rope(k, torch.tensor([20]), f)).sum()
    assert d1.item() == pytest.approx(d2.item(), abs=1e-5)


def test_llama3_frequencies_three_bands():
    sc = TINY_B["rope_scaling"]
    base = pl.rope_frequencies(32, 500000.0, None).double()
    got = pl.rope_frequencies(32, 500000.0, sc).double()
    kept = [j for j in range(16) if 2 * math.pi / base[j] < 64 / 4]
    slow = [j for j in range(16) if 2 * math.pi / base[j] > 64 / 1]
    mid = [j for j in range(16) if j not in kept and j not in slow]
    assert kept == [0, 1] and mid == [2] and slow == list(range(3, 16))
    assert torch.equal(got[kept], base[kept])
    assert torch.allclose(got[slow], base[slow] / 8, rtol=1e-6)
    assert base[2] / 8 < got[2] < base[2]


def test_attention_groups_mask_and_window():
    torch.manual_seed(0)
    T, nh, nkv, hd = 6, 4, 2, 8
    q, k, v = (torch.randn(T, h, hd, dtype=torch.float64) for h in (nh, nkv, nkv))
    out = pl.attention(q, k, v)
    # row 0 sees only key 0
    for a in range(nh):
        assert torch.allclose(out[0, a], v[0, a // 2])
    # head a by hand at the last row
    a, t = 3, T - 1
    s = (k[:, 1] @ q[t, a]) / math.sqrt(hd)
    p = torch.softmax(s, 0)
    assert torch.allclose(out[t, a], p @ v[:, 1])
    # a window of 2 sees the key itself and the one before
    outw = pl.attention(q, k, v, window=2)
    s2 = (k[t - 1:, 1] @ q[t, a]) / math.sqrt(hd)
    assert torch.allclose(outw[t, a], torch.softmax(s2, 0) @ v[t - 1:, 1])
    # changing a later key does not change earlier rows
    k2 = k.clone()
    k2[4] += 1
    assert torch.allclose(pl.attention(q, k2, v)[:4], out[:4])


def test_swiglu_by_hand():
    x = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    wg = torch.tensor([[0.5, 0.25]], dtype=torch.float64)
    wu = torch.tensor([[1.0, 1.0]], dtype=torch.float64)
    wd = torch.tensor([[2.0], [3.0]], dtype=torch.float64)
    g, u = 0.0, -1.0
    act = g / (1 + math.exp(-g)) * u
    assert torch.allclose(pl.swiglu(x, wg, wu, wd), torch.tensor([[2 * act, 3 * act]], dtype=torch.float64))


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B], ids=["A", "B"])
def test_forward_is_causal_and_precise(tmp_path, cfg):
    folder = make_model_folder(str(tmp_path / "m"), cfg, seed=11)
    c, w = pl.read_config(folder), pl.read_weights(folder)
    toks = random_tokens(40, cfg["vocab_size"], 1)
    full = pl.forward(c, w, toks)
    assert full.shape == (40, cfg["vocab_size"]) and torch.isfinite(full).all()
    assert torch.allclose(pl.forward(c, w, toks[:17]), full[:17], atol=1e-12)
    changed = toks[:30] + [(toks[30] + 1) % cfg["vocab_size"]] + toks[31:]
    again = pl.forward(c, w, changed)
    assert torch.allclose(again[:30], full[:30], atol=1e-12) and not torch.allclose(again[30:], full[30:])
    f32 = pl.forward(c, w, toks, dtype=torch.float32)
    assert (f32.double() - full).abs().max() / full.abs().max() < 2e-5


def test_tied_and_untied_heads(tmp_path):
    fa = make_model_folder(str(tmp_path / "a"), TINY_A, seed=2)
    wa = pl.read_weights(fa)
    assert "lm_head.weight" not in wa
    fb = make_model_folder(str(tmp_path / "b"), TINY_B, seed=2)
    wb = pl.read_weights(fb)
    c = pl.read_config(fb)
    toks = random_tokens(5, 320, 0)
    l1 = pl.forward(c, wb, toks)
    wb2 = dict(wb)
    wb2["lm_head.weight"] = wb["lm_head.weight"] * 2
    assert torch.allclose(pl.forward(c, wb2, toks), l1 * 2)


def test_sampling_distribution_and_choice():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 3.0])
    assert pl.argmax(torch.tensor([1.0, 5.0, 5.0, 2.0])) == 1
    p = pl.sample_probabilities(logits, 1.0, 1.0, 1.0, [])
    assert torch.allclose(p, torch.softmax(logits.double(), 0))
    p = pl.sample_probabilities(logits, 0.5, 0.9, 1.0, [])
    soft = torch.softmax(logits.double() / 0.5, 0)
    assert p[4] > 0 and p[0] > 0 and p[1] == 0 and p[2] == 0 and p[3] == 0  # 0.86 < 0.9 <= 0.86 + 0.12
    assert p[4].item() == pytest.approx((soft[4] / (soft[4] + soft[0])).item())
    pen = pl.sample_probabilities(logits, 1.0, 1.0, 2.0, [4, 4, 3])
    want = logits.double().clone()
    want[4] = want[4] / 4
    want[3] = want[3] * 2
    assert torch.allclose(pen, torch.softmax(want, 0))
    probs = torch.tensor([0.0, 0.25, 0.0, 0.75])
    assert pl.sample_index_order(probs, 0.1) == 1 and pl.sample_index_order(probs, 0.25) == 3
    assert pl.sample_index_order(probs, 0.9999) == 3


def test_greedy_generate_extends_itself(tmp_path):
    folder = make_model_folder(str(tmp_path / "m"), TINY_A, seed=4)
    c, w = pl.read_config(folder), pl.read_weights(folder)
    out = pl.greedy_generate(c, w, [5, 6, 7], 4)
    assert out[:2] == pl.greedy_generate(c, w, [5, 6, 7], 2)
    assert pl.greedy_generate(c, w, [5, 6, 7, out[0]], 3) == out[1:]
