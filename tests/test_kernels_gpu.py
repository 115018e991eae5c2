"""Each CUDA kernel alone against a plain float64 statement of the same
operation, at sizes other than the engine's test models use."""
import math
import random
from types import SimpleNamespace

import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def core():
    from infernum_b200.ops import core as c
    return c


def rel_err(got, ref):
    ref = ref.double().cpu()
    return float((got.double().cpu() - ref).abs().max() / max(ref.abs().max().item(), 1e-9))


TOL = {torch.float32: 3e-6, torch.bfloat16: 1.2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    c = core()
    table = torch.randn(77, 50).to(dtype).to(DEV)
    ids = torch.tensor([0, 76, 5, 5, 33], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 50, device=DEV)
    err = c.new_error_word(DEV)
    c.embed(ids, table, out, err)
    assert torch.equal(out.cpu(), table.float().cpu()[ids.long().cpu()])
    assert err.item() == 0
    c.embed(torch.tensor([3, 77], dtype=torch.int32, device=DEV), table, out[:2], err)
    assert err.item() == c.FLAG_BAD_TOKEN and out[1].abs().sum().item() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [50, 64, 333, 4096, 9000])
def test_add_rmsnorm(dtype, H):
    c = core()
    N, eps = 7, 3e-6
    res = torch.randn(N, H) * 3
    delta = torch.randn(N, H).to(dtype)
    w = (1 + 0.1 * torch.randn(H)).to(dtype)
    want_res = res.double() + delta.double()
    want = pl.rms_norm(want_res, w.double(), eps)
    r = res.clone().to(DEV)
    out = torch.empty(N, H, dtype=dtype, device=DEV)
    c.add_rmsnorm(r, delta.to(DEV), w.to(DEV), eps, out)
    assert rel_err(r, want_res) < 1e-6
    assert rel_err(out, want) < TOL[dtype]
    # without a delta, and with a float32 weight in a bfloat16 engine
    r2 = res.clone().to(DEV)
    c.add_rmsnorm(r2, None, w.float().to(DEV), eps, out)
    assert torch.equal(r2.cpu(), res)
    assert rel_err(out, pl.rms_norm(res.double(), w.double(), eps)) < TOL[dtype]
    # chosen rows only: compact output, residual untouched
    idx = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    r3 = res.clone().to(DEV)
    out3 = torch.empty(3, H, dtype=dtype, device=DEV)
    c.add_rmsnorm(r3, delta.to(DEV), w.to(DEV), eps, out3, row_idx=idx)
    assert torch.equal(r3.cpu(), res)
    assert rel_err(out3, want[[6, 0, 3]]) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul_and_residual_add(dtype):
    c = core()
    x = (torch.randn(9, 2 * 37) * 4).to(dtype)
    out = torch.empty(9, 37, dtype=dtype, device=DEV)
    c.silu_mul(x.to(DEV), out)
    g, u = x[:, :37].double(), x[:, 37:].double()
    assert rel_err(out, g / (1 + torch.exp(-g)) * u) < TOL[dtype]
    res = torch.randn(9, 37)
    r = res.clone().to(DEV)
    c.residual_add(r, out)
    assert rel_err(r, res.double() + out.double().cpu()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd, rd", [(16, 16), (48, 48), (64, 32), (128, 128)])
def test_rope_and_cache_write(dtype, hd, rd):
    c = core()
    from infernum_b200.parts.rope import rotary_inv_freq
    nh, nkv, N, ps, pages = 5, 2, 11, 4, 9
    scaling = {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
               "high_freq_factor": 4.0, "original_max_position_embeddings": 32}
    freqs = torch.tensor(rotary_inv_freq(rd, 10000.0, scaling), dtype=torch.float64).float()
    assert torch.equal(freqs, pl.rope_frequencies(rd, 10000.0, scaling))
    qkv = torch.randn(N, (nh + 2 * nkv) * hd).to(dtype)
    # two requests: rows 0..6 at positions 3..9 of request 0, rows 7..10 at 20..23 of request 1
    positions = torch.tensor(list(range(3, 10)) + list(range(20, 24)), dtype=torch.int32)
    row_entry = torch.tensor([0] * 7 + [1] * 4, dtype=torch.int32)
    tables = torch.tensor([[5, 2, 7, -1, -1, -1], [8, 0, 1, 3, 4, 6]], dtype=torch.int32)
    kp = torch.zeros(pages, nkv, ps, hd, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    err = c.new_error_word(DEV)
    d = qkv.clone().to(DEV)
    c.rope_append(d, positions.to(DEV), freqs.to(DEV), rd, nh, nkv, hd, row_entry.to(DEV),
                  tables.to(DEV), kp, vp, err)
    assert err.item() == 0
    x = qkv.double()
    q = x[:, : nh * hd].view(N, nh, hd)
    k = x[:, nh * hd: (nh + nkv) * hd].view(N, nkv, hd)
    v = x[:, (nh + nkv) * hd:].view(N, nkv, hd)

    def rot(t):
        return torch.cat([pl.rope(t[..., :rd], positions, freqs), t[..., rd:]], dim=-1)

    tol = TOL[dtype]
    got = d.cpu().double()
    assert rel_err(got[:, : nh * hd].view(N, nh, hd), rot(q)) < tol
    assert torch.equal(d[:, (nh + nkv) * hd:].cpu(), qkv[:, (nh + nkv) * hd:])
    written = 0
    for r in range(N):
        e, pos = int(row_entry[r]), int(positions[r])
        page, slot = int(tables[e, pos // ps]), pos % ps
        assert rel_err(kp[page, :, slot], rot(k)[r]) < tol
        assert torch.equal(vp[page, :, slot].cpu(), qkv[r, (nh + nkv) * hd:].view(nkv, hd))
        written += 1
    assert int((kp.abs().sum(dim=(1, 3)) > 0).sum()) == written  # nothing else was touched
    # a table entry outside the pool is reported, not followed
    bad = tables.clone()
    bad[0, 0] = 99
    c.rope_append(qkv.clone().to(DEV), positions.to(DEV), freqs.to(DEV), rd, nh, nkv, hd,
                  row_entry.to(DEV), bad.to(DEV), kp, vp, err)
    assert err.item() == c.FLAG_BAD_PAGE


@pytest.mark.parametrize("M, N, K", [(1, 1, 1), (3, 5, 7), (64, 64, 16), (65, 130, 33), (200, 77, 300)])
@pytest.mark.parametrize("dt", [(torch.float32,) * 3, (torch.bfloat16,) * 3,
                                (torch.bfloat16, torch.float32, torch.bfloat16),
                                (torch.bfloat16, torch.bfloat16, torch.float32)])
def test_gemm_plain(M, N, K, dt):
    c = core()
    a = torch.randn(M, K).to(dt[0])
    w = torch.randn(N, K).to(dt[1])
    out = torch.empty(M, N, dtype=dt[2], device=DEV)
    c.gemm_plain(a.to(DEV), w.to(DEV), out)
    assert rel_err(out, a.double() @ w.double().T) < TOL[dt[2]]
    if M > 1:  # a row does not depend on the others
        one = torch.empty(1, N, dtype=dt[2], device=DEV)
        c.gemm_plain(a[M - 1:].to(DEV), w.to(DEV), one)
        assert torch.equal(one[0], out[M - 1])


def test_argmax_lowest_index_wins():
    c = core()
    x = torch.randn(6, 1000)
    x[0, 17] = x[0, 900] = 50.0
    x[1, 999] = 60.0
    x[2, 0] = 70.0
    x[3] = -5.0  # all equal
    big = torch.randn(2, 128256)
    big[0, 128255] = 99.0
    big[1, 70000] = big[1, 3] = 99.0
    for t in (x, big):
        out = torch.empty(t.shape[0], dtype=torch.int32, device=DEV)
        c.argmax(t.to(DEV), out)
        assert out.tolist() == [pl.argmax(r) for r in t]


def pack_params(c, rows):
    p = torch.zeros(len(rows), c.SAMPLE_PARAM_FLOATS)
    n = torch.zeros(len(rows), dtype=torch.int32)
    for i, (t, tp, pen, u, nr) in enumerate(rows):
        p[i, :4] = torch.tensor([t, tp, pen, u])
        n[i] = nr
    p.view(torch.int32)[:, 4] = n
    return p.to(DEV)


@pytest.mark.parametrize("V, R", [(50, 24), (1000, 24), (5003, 24), (33000, 12), (128256, 6), (128256, 80),
                                  (200003, 6), (270001, 3)])
def test_sample_against_plain(V, R):
    """Rows of every width: one CTA a row, a row over 2, 4 and 8 CTAs of a
    cluster (few rows: 16 candidate thresholds a pass; many rows: 4), and
    beyond 262,144 tokens the kernel that reads its row once per pass."""
    c = core()
    rng = random.Random(V)
    logits = torch.randn(R, V, generator=torch.Generator().manual_seed(V)) * 3
    rows, recents = [], torch.zeros(R, 8, dtype=torch.int32)
    for i in range(R):
        nr = rng.randint(0, 8)
        recents[i, :nr] = torch.tensor([rng.randrange(V) for _ in range(nr)], dtype=torch.int32)
        if nr >= 2:
            recents[i, 1] = recents[i, 0]  # a token that occurs twice is penalised twice
        rows.append((rng.choice([0.3, 0.7, 1.0, 1.5]), rng.choice([0.5, 0.9, 0.95, 1.0]),
                     rng.choice([1.0, 1.1, 1.3]), rng.random(), nr))
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    c.sample(logits.clone().to(DEV), pack_params(c, rows), recents.to(DEV), out)
    exact = 0
    for i, (t, tp, pen, u, nr) in enumerate(rows):
        # The plain distribution in 64-bit, and the place of the kernel's token in it.  The
        # kernel works in 32-bit: its sums are off by rounding, and a token at the very edge
        # of the nucleus (one of many of nearly the same, tiny probability in a wide
        # vocabulary) may be in or out.  Either moves the cumulative distribution by some
        # 1e-6, so the token must be the one whose interval holds u to within 1e-5.
        probs = pl.sample_probabilities(logits[i], t, tp, pen, recents[i, :nr].tolist())
        got = int(out[i].item())
        cdf = torch.cumsum(probs, 0)
        lo = float(cdf[got - 1]) if got > 0 else 0.0
        hi = float(cdf[got])
        assert lo - 1e-5 <= u < hi + 1e-5, f"row {i}: {rows[i]} -> {got}, interval [{lo}, {hi})"
        if probs[got] == 0:  # only a token at the edge: as probable as the least probable one kept
            full = pl.sample_probabilities(logits[i], t, 1.0, pen, recents[i, :nr].tolist())
            assert tp < 1.0 and full[got] >= (1 - 1e-4) * full[probs > 0].min(), f"row {i}: {rows[i]} -> {got}"
        exact += int(got == pl.sample_index_order(probs, u))
    assert exact >= R // 2  # (most rows are nowhere near an edge)


def test_sample_distribution_over_many_draws():
    c = core()
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 1.5, -3.0])
    n = 4000
    us = (torch.arange(n) + 0.5) / n
    rows = [(0.8, 0.9, 1.0, float(u), 0) for u in us]
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    c.sample(logits.repeat(n, 1).to(DEV), pack_params(c, rows), None, out)
    freq = torch.bincount(out.cpu().long(), minlength=6).double() / n
    want = pl.sample_probabilities(logits, 0.8, 0.9, 1.0, [])
    assert (freq - want).abs().max() < 2e-3 and freq[want == 0].sum() == 0


# --------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------
def paged_case(seqs_len, q_rows, nh, nkv, hd, ps, dtype, seed, extra_pages=5, scale_key=None, poison=False):
    """Requests with ``seqs_len[i]`` cached+new tokens of which the last
    ``q_rows[i]`` are this step's rows.  Pages are handed out in a shuffled
    order.  Returns what the kernels take plus the plain result.  ``poison``:
    every slot of the pools that holds no key of a request - the rest of a
    request's last page, pages nobody holds (page 0 among them) - is NaN, as a
    request that went wrong might have left them."""
    g = torch.Generator().manual_seed(seed)
    E = len(seqs_len)
    n_pages = sum(-(-L // ps) for L in seqs_len) + extra_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    MB = max(-(-L // ps) for L in seqs_len)
    tables = torch.full((E, MB), -1, dtype=torch.int32)
    kp = torch.randn(n_pages, nkv, ps, hd, generator=g).to(dtype)  # stale data in unused slots
    vp = torch.randn(n_pages, nkv, ps, hd, generator=g).to(dtype)
    if poison:
        perm.remove(0)  # nobody holds page 0, which kernels may fetch in place of a missing table entry
        kp.fill_(float("nan"))
        vp.fill_(float("nan"))
    qs, refs, positions, row_entry, cu, q_start = [], [], [], [], [0], []
    for e, (L, n) in enumerate(zip(seqs_len, q_rows)):
        k = torch.randn(L, nkv, hd, generator=g).to(dtype)
        v = torch.randn(L, nkv, hd, generator=g).to(dtype)
        q = torch.randn(L, nh, hd, generator=g).to(dtype)
        if scale_key is not None:  # one far key stands out for the last query
            j = scale_key if scale_key >= 0 else L + scale_key
            k[j] = k[j] * 0 + q[L - 1, :: nh // nkv][:nkv] * 4.0
        for i in range(-(-L // ps)):
            tables[e, i] = perm.pop()
            lo, hi = i * ps, min(L, (i + 1) * ps)
            kp[tables[e, i], :, : hi - lo] = k[lo:hi].transpose(0, 1)
            vp[tables[e, i], :, : hi - lo] = v[lo:hi].transpose(0, 1)
        refs.append((q.double(), k.double(), v.double(), L - n))
        qs.append(q[L - n:].reshape(n, nh * hd))
        positions += list(range(L - n, L))
        row_entry += [e] * n
        cu.append(cu[-1] + n)
        q_start.append(L - n)
    q_all = torch.cat(qs)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    ctx = SimpleNamespace(n_rows=q_all.shape[0], n_entries=E, positions=i32(positions),
                          row_entry=i32(row_entry), cu_rows=i32(cu), q_start=i32(q_start),
                          host_cu_rows=cu, max_rows_per_entry=max(q_rows), max_kv_len=max(seqs_len),
                          scratch={})
    return q_all.to(DEV), kp.to(DEV), vp.to(DEV), tables.to(DEV), ctx, refs


def plain_result(refs, window=0):
    outs = []
    for q, k, v, start in refs:
        o = pl.attention(q, k, v, window=window)
        outs.append(o[start:].reshape(o.shape[0] - start, -1))
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, hd, ps, window", [
    (4, 2, 16, 4, 0), (3, 1, 32, 8, 0), (6, 6, 48, 16, 0), (8, 2, 128, 16, 0), (5, 5, 80, 2, 0),
    (4, 1, 64, 4, 7), (2, 2, 256, 32, 0), (40, 1, 16, 4, 0),
])
def test_attention_plain(dtype, nh, nkv, hd, ps, window):
    c = core()
    q, kp, vp, tables, ctx, refs = paged_case([37, 1, 64, 5], [37, 1, 3, 2], nh, nkv, hd, ps, dtype, 1)
    out = torch.empty(q.shape[0], nh * hd, dtype=dtype, device=DEV)
    err = c.new_error_word(DEV)
    c.attention_plain(q, kp, vp, out, ctx.positions, ctx.row_entry, tables, nh,
                      1 / math.sqrt(hd), window, err)
    assert err.item() == 0
    assert rel_err(out, plain_result(refs, window)) < (2e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_plain_finds_a_far_key(dtype):
    """Among hundreds of keys one far key carries the answer."""
    c = core()
    for key in (0, 3, -300, 129):
        q, kp, vp, tables, ctx, refs = paged_case([700], [1], 4, 2, 32, 16, dtype, 2, scale_key=key)
        out = torch.empty(1, 4 * 32, dtype=dtype, device=DEV)
        c.attention_plain(q, kp, vp, out, ctx.positions, ctx.row_entry, tables, 4,
                          1 / math.sqrt(32), 0, c.new_error_word(DEV))
        want = plain_result(refs)
        j = key if key >= 0 else 700 + key
        v_far = refs[0][2][j]  # [nkv, hd]
        assert (want.view(4, 32)[0] - v_far[0]).abs().max() < 0.2  # the answer is that key's value
        # scores reach |s| ~ 23 here, and exp(s) carries the rounding of s itself:
        # relative error ~ |s| * 2^-23 * (a few) ~ 1e-5 in float32
        assert rel_err(out, want) < (3e-5 if dtype == torch.float32 else 1e-2)


MMA_CASES = [
    # nh, nkv, hd, ps, window, lengths, rows
    (4, 2, 16, 4, 0, [37, 1, 64, 5], [37, 1, 3, 2]),        # mixed: tile and split entries
    (3, 1, 32, 8, 0, [100, 130], [100, 2]),                  # G = 3 (not a power of two)
    (8, 2, 128, 16, 0, [300, 77, 513], [1, 1, 1]),           # pure decode, slices
    (8, 2, 128, 16, 0, [257, 64], [257, 64]),                # whole prompts
    (6, 6, 48, 16, 0, [90, 33], [40, 33]),                   # G = 1, a portion with a cached prefix
    (32, 1, 64, 16, 0, [150, 20], [1, 20]),                  # G = 32 > 16: head sub-blocks
    (4, 1, 64, 4, 9, [80, 30, 12], [80, 1, 3]),              # a window
    (2, 2, 256, 32, 0, [70], [70]),
    (5, 5, 80, 2, 0, [45, 9], [5, 9]),
    (4, 4, 112, 16, 0, [130], [1]),
]


@pytest.mark.parametrize("case", MMA_CASES, ids=[f"nh{c[0]}kv{c[1]}hd{c[2]}ps{c[3]}w{c[4]}r{max(c[6])}" for c in MMA_CASES])
def test_attention_mma_against_plain(case):
    from infernum_b200.ops import attention_fast
    from infernum_b200.parts.base import Runtime
    nh, nkv, hd, ps, window, lens, rows = case
    c = core()
    q, kp, vp, tables, ctx, refs = paged_case(lens, rows, nh, nkv, hd, ps, torch.bfloat16, 3)
    rt = Runtime(torch.device(DEV), torch.bfloat16, err=c.new_error_word(DEV))
    out = torch.full((q.shape[0], nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert attention_fast.run(q, kp, vp, out, ctx, tables, nh, 1 / math.sqrt(hd), window, rt)
    assert rt.err.item() == 0
    want = plain_result(refs, window)
    assert torch.isfinite(out).all()
    assert rel_err(out, want) < 1e-2
    twin = torch.empty_like(out)
    c.attention_plain(q, kp, vp, twin, ctx.positions, ctx.row_entry, tables, nh,
                      1 / math.sqrt(hd), window, rt.err)
    assert rel_err(out, twin.double()) < 1e-2


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
def test_attention_mma_slices_agree(splits):
    from infernum_b200.ops import attention_fast
    from infernum_b200.parts.base import Runtime
    c = core()
    nh, nkv, hd = 8, 2, 128
    q, kp, vp, tables, ctx, refs = paged_case([700, 64, 65, 1], [1, 1, 1, 1], nh, nkv, hd, 16,
                                              torch.bfloat16, 4, scale_key=0)
    ctx.attention_mode = (2, splits)
    rt = Runtime(torch.device(DEV), torch.bfloat16, err=c.new_error_word(DEV))
    out = torch.full((4, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert attention_fast.run(q, kp, vp, out, ctx, tables, nh, 1 / math.sqrt(hd), 0, rt)
    assert rel_err(out, plain_result(refs)) < 1e-2


def test_attention_mma_edges_of_tiles_and_pages():
    """Lengths around the 64-key tile and the page edge, one query each, with
    the last key standing out: a tile or page that is dropped or read twice
    changes the answer."""
    from infernum_b200.ops import attention_fast
    from infernum_b200.parts.base import Runtime
    c = core()
    nh, nkv, hd, ps = 4, 2, 64, 16
    for L in (1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 191, 193):
        for n in (1, min(L, 3), L):
            q, kp, vp, tables, ctx, refs = paged_case([L], [n], nh, nkv, hd, ps, torch.bfloat16,
                                                      L * 7 + n, scale_key=-1)
            rt = Runtime(torch.device(DEV), torch.bfloat16, err=c.new_error_word(DEV))
            out = torch.full((n, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
            assert attention_fast.run(q, kp, vp, out, ctx, tables, nh, 1 / math.sqrt(hd), 0, rt)
            assert rel_err(out, plain_result(refs)) < 1e-2, (L, n)


@pytest.mark.parametrize("hd, ps, window", [
    (64, 8, 0), (128, 8, 0), (128, 16, 0), (128, 32, 0), (64, 64, 0), (128, 128, 0), (128, 256, 0),
    (128, 16, 40), (64, 32, 100), (128, 8, 64), (64, 128, 130),
])
@pytest.mark.parametrize("splits", [1, 3, 12])
def test_attention_split_by_tma_and_by_cp_async(hd, ps, window, splits):
    """Split mode fetches whole pages by TMA where it can.  What a page holds
    beyond the request's last key, and pages that a window has given back, must
    not reach the result: they are poisoned here with NaN.  Both ways of
    fetching give the plain result."""
    from infernum_b200.ops import attention_fast
    from infernum_b200.parts.base import Runtime
    c = core()
    nh, nkv = 8, 2
    lens = [1, 63, 64, 65, 200, 517]
    q, kp, vp, tables, ctx, refs = paged_case(lens, [1] * len(lens), nh, nkv, hd, ps, torch.bfloat16,
                                              hd + ps + window, scale_key=0 if window == 0 else -1)
    tables_h = tables.cpu()
    used = set()
    for e, L in enumerate(lens):
        n_pages = -(-L // ps)
        kv_min = max(0, L - window) if window else 0
        for i in range(n_pages):
            page = int(tables_h[e, i])
            used.add(page)
            hi = min(L, (i + 1) * ps) - i * ps
            kp[page, :, hi:] = float("nan")
            vp[page, :, hi:] = float("nan")
            if (i + 1) * ps <= kv_min:  # the window has passed this page: given back
                kp[page] = float("nan")
                vp[page] = float("nan")
                tables_h[e, i] = -1
    for page in range(kp.shape[0]):
        if page not in used:
            kp[page] = float("nan")
            vp[page] = float("nan")
    tables = tables_h.to(DEV)
    want = plain_result(refs, window)
    outs = []
    for copy in ("tma", "cp.async"):
        ctx.attention_mode = (2, splits)
        rt = Runtime(torch.device(DEV), torch.bfloat16, err=c.new_error_word(DEV), options={"split_copy": copy})
        out = torch.full((len(lens), nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert attention_fast.run(q, kp, vp, out, ctx, tables, nh, 1 / math.sqrt(hd), window, rt)
        assert rt.err.item() == 0, copy
        assert torch.isfinite(out).all(), copy
        assert rel_err(out, want) < 1e-2, copy
        outs.append(out)
    assert rel_err(outs[0], outs[1].double()) < 4e-3


# --------------------------------------------------------------------------
# the tcgen05 matrix product
# --------------------------------------------------------------------------
@pytest.mark.parametrize("T, N, K, splits", [
    (1, 128, 64, 1), (16, 128, 256, 1), (8, 200, 120, 1), (33, 333, 200, 1), (64, 640, 1024, 2),
    (100, 512, 1024, 1), (300, 256, 512, 1), (8, 1024, 4096, 8), (3, 320, 96, 1), (30, 300, 2048, 8),
    (17, 130, 1000, 4), (257, 384, 264, 1),
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05(T, N, K, splits, out_dtype):
    from infernum_b200.ops import gemm_tc
    g = torch.Generator().manual_seed(T * 1000 + N)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    out = torch.full((T, N), float("nan"), dtype=out_dtype, device=DEV)
    gemm_tc.gemm_tc(x.to(DEV), w.to(DEV), out, splits=splits)
    assert gemm_tc.error_flags(DEV) == 0
    assert rel_err(out, x.double() @ w.double().T) < (5e-3 if out_dtype == torch.bfloat16 else 2e-6)
    # a row of tokens does not depend on the others in the batch
    if T > 1:
        one = torch.empty(1, N, dtype=out_dtype, device=DEV)
        gemm_tc.gemm_tc(x[T - 1:].contiguous().to(DEV), w.to(DEV), one, splits=splits)
        assert rel_err(one[0], out[T - 1]) < 1e-6 if out_dtype == torch.float32 else True


def test_gemm_tcgen05_takes_strided_rows_and_refuses_what_tma_cannot_fetch():
    from infernum_b200.ops import gemm_tc
    big = torch.randn(10, 512).to(torch.bfloat16).to(DEV)
    x = big[:, :256]  # row stride 512, 256 columns
    w = torch.randn(140, 256).to(torch.bfloat16).to(DEV)
    out = torch.empty(10, 140, dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_tc(x, w, out)
    assert rel_err(out, x.double().cpu() @ w.double().cpu().T) < 5e-3
    assert not gemm_tc.eligible(big[:, :250], w[:, :250], out)  # K not a multiple of 8
    assert not gemm_tc.eligible(big[:, 1:257], w, out)  # base not 16-byte aligned


@pytest.mark.parametrize("T, I, K", [(1, 128, 64), (8, 256, 512), (33, 192, 200), (64, 1024, 1024)])
def test_gemm_tcgen05_with_swiglu_epilogue(T, I, K):
    """Weight rows interleaved 64 gates / 64 ups per tile; the epilogue stores silu(gate) * up."""
    from infernum_b200.ops import gemm_tc
    g = torch.Generator().manual_seed(I + T)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    wg = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    wu = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    w = torch.stack([wg.view(I // 64, 64, K), wu.view(I // 64, 64, K)], dim=1).reshape(2 * I, K)
    out = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_tc(x.to(DEV), w.contiguous().to(DEV), out, splits=1, swiglu=True)
    assert gemm_tc.error_flags(DEV) == 0
    gate, up = x.double() @ wg.double().T, x.double() @ wu.double().T
    want = gate / (1 + torch.exp(-gate)) * up
    assert rel_err(out, want) < 6e-3
    # the stand-alone kernel reads the same interleaved layout
    c = core()
    gu = (x.double() @ w.double().T).to(torch.bfloat16).to(DEV)
    out2 = torch.empty(T, I, dtype=torch.bfloat16, device=DEV)
    c.silu_mul(gu, out2, block=64)
    assert rel_err(out2, want) < 2e-2



# --------------------------------------------------------------------------
# the matrix product on pairs of SMs (prompts)
# --------------------------------------------------------------------------
@pytest.mark.parametrize("T, N, K", [
    (256, 256, 64), (300, 392, 200), (129, 640, 1000), (65, 128, 72), (1000, 1024, 520), (2048, 4096, 256),
    (515, 6000, 136),
])
@pytest.mark.parametrize("tiling", [None, (32, 1 << 20, 32), (112, 1, 176), (256, 2, 240), (256, 0, 144)])
def test_gemm_pair(T, N, K, tiling):
    """Every way of cutting the weight rows gives the product; widths that are no
    divisor of N, token counts that are no multiple of the tile, a short K."""
    from infernum_b200.ops import gemm_tc
    g = torch.Generator().manual_seed(T * 1000 + N)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_pair(x.to(DEV), w.to(DEV), out, tiling=tiling)
    assert gemm_tc.error_flags(DEV) == 0
    assert rel_err(out, x.double() @ w.double().T) < 5e-3
    # rounding apart, it is the product of the kernel for few tokens
    few = torch.empty(min(T, 64), N, dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_tc(x[:few.shape[0]].contiguous().to(DEV), w.to(DEV), few, splits=1)
    assert rel_err(out[:few.shape[0]], few.double().cpu()) < 5e-3


@pytest.mark.parametrize("T, group", [(1300, 1), (1300, 4), (1300, 5), (1300, 6), (2048, 3), (700, 2)])
@pytest.mark.parametrize("tiling", [None, (256, 2, 144), (128, 1 << 20, 128), (256, 0, 192)])
def test_gemm_pair_token_groups(T, group, tiling):
    """The tokens walked in groups of token tiles, even and uneven ones, beside a
    second region that runs over all tokens: every output element is written, once."""
    from infernum_b200.ops import gemm_tc
    N, K = 1000, 136
    g = torch.Generator().manual_seed(T + group)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_pair(x.to(DEV), w.to(DEV), out, tiling=tiling, token_group=group)
    assert gemm_tc.error_flags(DEV) == 0
    assert rel_err(out, x.double() @ w.double().T) < 5e-3
    whole = torch.empty_like(out)
    gemm_tc.gemm_pair(x.to(DEV), w.to(DEV), whole, tiling=tiling, token_group=1 << 20)
    assert torch.equal(out, whole)  # the order of the tiles changes no value


@pytest.mark.parametrize("T, I, K", [(256, 128, 64), (300, 192, 200), (700, 1024, 1024), (64, 320, 520)])
@pytest.mark.parametrize("tiling", [None, (128, 1 << 20, 128), (256, 1, 128), (128, 3, 256)])
def test_gemm_pair_with_swiglu_epilogue(T, I, K, tiling):
    from infernum_b200.ops import gemm_tc
    g = torch.Generator().manual_seed(I + T)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    wg = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    wu = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    w = torch.stack([wg.view(I // 64, 64, K), wu.view(I // 64, 64, K)], dim=1).reshape(2 * I, K)
    out = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_pair(x.to(DEV), w.contiguous().to(DEV), out, swiglu=True, tiling=tiling)
    assert gemm_tc.error_flags(DEV) == 0
    gate, up = x.double() @ wg.double().T, x.double() @ wu.double().T
    want = gate / (1 + torch.exp(-gate)) * up
    assert rel_err(out, want) < 6e-3


def test_gemm_pair_refuses_widths_it_cannot_run():
    from infernum_b200.errors import KernelError
    from infernum_b200.ops import gemm_tc
    x = torch.zeros(256, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(256, 64, dtype=torch.bfloat16, device=DEV)
    out = torch.empty(256, 256, dtype=torch.bfloat16, device=DEV)
    for tiling in [(264, 1, 256), (256, 1, 24), (250, 1, 256)]:
        with pytest.raises(KernelError):
            gemm_tc.gemm_pair(x, w, out, tiling=tiling)
    with pytest.raises(KernelError):  # the activation wants whole blocks of 64 gates and 64 ups
        gemm_tc.gemm_pair(x, w, out[:, :128], swiglu=True, tiling=(192, 1, 128))


def test_pair_tiling_covers_the_weight_rows():
    """The chosen cut is one the kernel accepts and never costs more, by the
    chooser's own measure, than full-width tiles."""
    from infernum_b200.ops import gemm_tc
    for T in (200, 256, 512, 1000, 2048, 5000):
        for N, sw in ((4096, False), (6144, False), (28672, True), (1000, False), (128256, False), (384, True)):
            bn_a, cols_a, bn_b = gemm_tc.choose_pair_tiling(T, N, 148, sw)
            step = 128 if sw else 16
            assert bn_a % step == 0 and bn_b % step == 0 and 32 <= bn_a <= 256 and 32 <= bn_b <= 256
            assert 0 <= cols_a <= -(-N // bn_a)


TC_CASES = [
    # nh, nkv, hd, ps, lengths, rows
    (8, 2, 128, 16, [257, 64], [257, 64]),           # whole prompts
    (8, 2, 128, 16, [300, 77, 513, 90], [1, 40, 200, 2]),   # prompt portions beside decoded tokens
    (4, 4, 64, 8, [130, 65], [130, 33]),             # G = 1, head size 64, pages of 8
    (16, 2, 64, 32, [100], [100]),                   # G = 8
    (32, 1, 128, 16, [70, 200], [70, 9]),            # G = 32
    (8, 2, 128, 64, [1000], [1000]),                 # pages of 64, many tiles
]


@pytest.mark.parametrize("poison", [False, True], ids=["stale", "nan"])
@pytest.mark.parametrize("case", TC_CASES, ids=[f"nh{c[0]}kv{c[1]}hd{c[2]}ps{c[3]}r{max(c[5])}" for c in TC_CASES])
def test_attention_tcgen05_against_plain(case, poison):
    """``poison``: what pages hold beyond a request's last key, and pages it does
    not hold, are NaN (values only, nothing faults): masked keys have P = 0, but
    0 x NaN is NaN in the product P V unless those rows of V are cleared."""
    from infernum_b200.ops import attention_fast
    from infernum_b200.parts.base import Runtime
    nh, nkv, hd, ps, lens, rows = case
    c = core()
    q, kp, vp, tables, ctx, refs = paged_case(lens, rows, nh, nkv, hd, ps, torch.bfloat16, 11, poison=poison)
    # queries sit in rows as wide as the fused qkv rows of the engine
    wide = torch.zeros(q.shape[0], (nh + 2 * nkv) * hd, dtype=torch.bfloat16, device=DEV)
    wide[:, : nh * hd] = q
    out = torch.full((q.shape[0], nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert attention_fast.tc_eligible(wide, kp, out, nh, 0)
    rt = Runtime(torch.device(DEV), torch.bfloat16, err=c.new_error_word(DEV))
    assert attention_fast.run(wide, kp, vp, out, ctx, tables, nh, 1 / math.sqrt(hd), 0, rt)
    assert rt.err.item() == 0
    assert torch.isfinite(out).all()
    assert rel_err(out, plain_result(refs)) < 1e-2
    # and against the mma.sync kernel on the same inputs
    rt2 = Runtime(torch.device(DEV), torch.bfloat16, err=c.new_error_word(DEV),
                  options={"prompt_attention": "mma"})
    out2 = torch.empty_like(out)
    assert attention_fast.run(wide, kp, vp, out2, ctx, tables, nh, 1 / math.sqrt(hd), 0, rt2)
    assert rel_err(out, out2.double()) < 1e-2


@pytest.mark.parametrize("splits", [2, 4])
@pytest.mark.parametrize("nh, nkv, hd, ps, lens, rows", [
    (8, 2, 128, 16, [1500, 700], [200, 130]),     # portions after long cached prefixes
    (8, 2, 128, 16, [257, 64, 100], [257, 64, 3]),  # whole prompts, fewer key tiles than slices, a short entry
    (4, 4, 64, 8, [900], [77]),                     # head size 64, pages of 8
    (32, 1, 128, 64, [640, 2000], [9, 300]),        # G = 32, pages of 64
])
def test_attention_tcgen05_with_key_slices(nh, nkv, hd, ps, lens, rows, splits):
    """The keys of a row tile shared out over 2 or 4 CTAs of a cluster and merged
    through distributed shared memory: the result is that of one CTA, also when a
    slice gets no key tile at all, and one key that carries the answer is found
    in whichever slice it lies."""
    from infernum_b200.ops import attention_fast
    from infernum_b200.parts.base import Runtime
    c = core()
    for far in (None, 0, 33, -1):
        q, kp, vp, tables, ctx, refs = paged_case(lens, rows, nh, nkv, hd, ps, torch.bfloat16, 17,
                                                  scale_key=far, poison=(far == 33))
        wide = torch.zeros(q.shape[0], (nh + 2 * nkv) * hd, dtype=torch.bfloat16, device=DEV)
        wide[:, : nh * hd] = q
        outs = []
        for s in (1, splits):
            ctx.prompt_splits = s
            rt = Runtime(torch.device(DEV), torch.bfloat16, err=c.new_error_word(DEV))
            out = torch.full((q.shape[0], nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
            assert attention_fast.run(wide, kp, vp, out, ctx, tables, nh, 1 / math.sqrt(hd), 0, rt)
            assert rt.err.item() == 0 and torch.isfinite(out).all()
            assert rel_err(out, plain_result(refs)) < 1e-2, (far, s)
            outs.append(out)
        # both are rounded to bfloat16: one unit in the last place of the largest value apart at most
        assert rel_err(outs[1], outs[0].double()) < 2 ** -7, far


def test_attention_tcgen05_far_key_and_edges():
    """One key carries the answer, at tile and page edges of a long prompt."""
    from infernum_b200.ops import attention_fast
    from infernum_b200.parts.base import Runtime
    c = core()
    nh, nkv, hd, ps = 8, 2, 128, 16
    for L, key in ((700, 0), (700, 63), (700, 64), (700, 127), (513, 511), (300, -1), (65, 64)):
        q, kp, vp, tables, ctx, refs = paged_case([L], [L], nh, nkv, hd, ps, torch.bfloat16, L + key + 5,
                                                  scale_key=key)
        out = torch.full((L, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        rt = Runtime(torch.device(DEV), torch.bfloat16, err=c.new_error_word(DEV))
        assert attention_fast.run(q, kp, vp, out, ctx, tables, nh, 1 / math.sqrt(hd), 0, rt)
        assert rt.err.item() == 0
        assert rel_err(out, plain_result(refs)) < 1e-2, (L, key)


# --------------------------------------------------------------------------
# a wait that runs out
# --------------------------------------------------------------------------
def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """Every wait of the kernels on a barrier is bounded in time.  Here a probe
    kernel waits 30 ms for a barrier on which nobody arrives: it returns, the
    error word says that a wait ran out and which one, and the next kernel runs
    as if nothing had happened."""
    import time
    from infernum_b200.errors import KernelError
    c = core()
    err = c.new_error_word(DEV)
    t0 = time.perf_counter()
    c.wait_probe(err, 30.0, 7)
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    assert 0.02 < took < 5.0
    flags = int(err.item())
    assert flags & c.FLAG_WAIT_TIMEOUT
    assert "prompt attention: MMA issuer" in c.describe_flags(flags)
    assert "a device-side wait ran out" in c.describe_flags(flags)
    # a wait of a matrix product is named the same way
    err.zero_()
    c.wait_probe(err, 30.0, c.TIMEOUT_SITES.index("product on SM pairs: epilogue"))
    torch.cuda.synchronize()
    assert "product on SM pairs: epilogue" in c.describe_flags(int(err.item()))
    assert "prompt attention" not in c.describe_flags(int(err.item()))
    with pytest.raises(KernelError):
        c.wait_probe(err, 5000.0, 0)  # longer than a second is refused
    x = torch.randn(4, 64).to(DEV)
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    c.argmax(x, out)
    assert out.tolist() == x.argmax(dim=1).tolist()
