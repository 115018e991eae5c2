"""Each part alone against the plain function it stands for, and a model whose
schedule runs a layer twice and shares a cache."""
import math

import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = {torch.float32: 5e-6, torch.bfloat16: 2e-2}


def runtime(dtype, **options):
    from infernum_b200.ops import core
    from infernum_b200.parts.base import Runtime
    return Runtime(DEV, dtype, err=core.new_error_word(DEV), options=options)


def rel_err(got, ref):
    ref = ref.double().cpu()
    return float((got.double().cpu() - ref).abs().max() / max(ref.abs().max().item(), 1e-9))


def weights_for(part, dtype, seed=0):
    from infernum_b200.weights.random_init import random_tensors
    return random_tensors(part.weight_specs(), seed, DEV, dtype)


def step_ctx(cache, requests):
    """requests: list of (RequestCache, n_new tokens).  Builds the step inputs
    the way the engine does, with pages reserved."""
    from infernum_b200.engine.step import ModelRunner, StepEntry
    from types import SimpleNamespace
    fake = SimpleNamespace(rt=runtime(torch.float32), spec=SimpleNamespace(vocab_size=1 << 30))
    runner = ModelRunner(fake, cache)
    entries = [StepEntry(rc, [0] * n, []) for rc, n in requests]
    runner.reserve(entries)
    return runner._build(entries)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from infernum_b200.parts import NORMS, ResidualStream
    rt = runtime(dtype)
    norm = NORMS.get("rmsnorm")({"hidden_size": 72, "eps": 2e-6, "weight": "w"}, rt)
    w = weights_for(norm, dtype)
    norm.bind(w)
    x = torch.randn(5, 72, device=DEV)
    d = torch.randn(5, 72, device=DEV).to(dtype)
    stream = ResidualStream(x.clone())
    stream.push(d)
    out = norm.forward(stream)
    assert stream.pending is None
    assert rel_err(stream.residual, x.double() + d.double()) < 1e-6
    assert rel_err(out, pl.rms_norm(x.double() + d.double(), w["w"].double(), 2e-6)) < TOL[dtype]
    assert rel_err(norm.apply(x), pl.rms_norm(x.double(), w["w"].double(), 2e-6)) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotary_part(dtype):
    from infernum_b200.parts import POSITION_ENCODINGS
    rt = runtime(dtype)
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
               "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    rope = POSITION_ENCODINGS.get("rotary")({"head_dim": 48, "theta": 5e5, "scaling": scaling}, rt)
    q = torch.randn(6, 5, 48).to(dtype).to(DEV)
    k = torch.randn(6, 2, 48).to(dtype).to(DEV)
    pos = torch.tensor([0, 1, 63, 64, 200, 4000], dtype=torch.int32, device=DEV)
    q0, k0 = q.clone(), k.clone()
    rope.apply(q, k, pos)
    f = pl.rope_frequencies(48, 5e5, scaling)
    assert torch.equal(rope.inv_freq.cpu(), f)
    assert rel_err(q, pl.rope(q0.double().cpu(), pos.cpu(), f)) < TOL[dtype]
    assert rel_err(k, pl.rope(k0.double().cpu(), pos.cpu(), f)) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from infernum_b200.parts import FEED_FORWARDS
    rt = runtime(dtype)
    ffn = FEED_FORWARDS.get("swiglu")({"hidden_size": 40, "intermediate_size": 104, "prefix": "m."}, rt)
    w = weights_for(ffn, dtype)
    for k in w:
        w[k] = (w[k].float() * 8).to(dtype)
    ffn.bind(w)
    x = torch.randn(9, 40).to(dtype).to(DEV)
    want = pl.swiglu(x.double().cpu(), *(w[f"m.{n}_proj.weight"].double().cpu() for n in ("gate", "up", "down")))
    assert rel_err(ffn.forward(x), want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("impl", ["auto", "plain"])
@pytest.mark.parametrize("nh, nkv, hd, window", [(4, 2, 16, 0), (3, 1, 32, 0), (6, 3, 48, 11)])
def test_attention_part_in_portions(dtype, impl, nh, nkv, hd, window):
    """The attention part fed a sequence in portions through a real cache
    equals plain attention over the whole sequence."""
    from infernum_b200.cache import CacheManager
    from infernum_b200.models.model import CacheNeed
    from infernum_b200.parts import MIXERS
    rt = runtime(dtype, attention=impl)
    H, T = 56, 45
    params = {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
              "window": window, "prefix": "a.",
              "position": {"kind": "rotary", "params": {"head_dim": hd, "theta": 10000.0}}}
    attn = MIXERS.get("attention")(params, rt)
    w = weights_for(attn, dtype)
    for k in w:
        w[k] = (w[k].float() * 10).to(dtype)
    attn.bind(w)
    cache = CacheManager([CacheNeed(0, attn.cache_spec(), None, None)], page_size=4, num_pages=16,
                         max_requests=2, dtype=dtype, device=DEV)
    x = torch.randn(T, H).to(dtype).to(DEV)
    rc = cache.admit("r")
    outs, pos = [], 0
    for n in [7, 1, 2, 13, 1, 1, 20]:
        ctx = step_ctx(cache, [(rc, n)])
        outs.append(attn.forward(x[pos: pos + n], ctx, cache.layer_caches[0]))
        cache.commit(rc, n)
        pos += n
    got = torch.cat(outs)
    xd = x.double().cpu()
    W = {k: v.double().cpu() for k, v in w.items()}
    f = pl.rope_frequencies(hd, 10000.0, None)
    p = torch.arange(T)
    q = pl.rope((xd @ W["a.q_proj.weight"].T).view(T, nh, hd), p, f)
    k = pl.rope((xd @ W["a.k_proj.weight"].T).view(T, nkv, hd), p, f)
    v = (xd @ W["a.v_proj.weight"].T).view(T, nkv, hd)
    want = pl.attention(q, k, v, window=window).reshape(T, nh * hd) @ W["a.o_proj.weight"].T
    assert rt.err.item() == 0
    assert rel_err(got, want) < TOL[dtype]
    if window:
        assert sum(1 for page in rc.tables[0] if page == -1) > 0  # pages behind the window came back


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from infernum_b200.parts import EMBEDDINGS, HEADS
    rt = runtime(dtype)
    emb = EMBEDDINGS.get("token_embedding")({"vocab_size": 90, "hidden_size": 24, "weight": "e"}, rt)
    head = HEADS.get("linear_head")({"vocab_size": 90, "hidden_size": 24, "weight": "h", "tied_to": "e"}, rt)
    assert head.weight_specs() == {}
    w = weights_for(emb, dtype)
    emb.bind(w)
    head.bind(w)
    ids = torch.tensor([3, 89, 0], dtype=torch.int32, device=DEV)
    h = emb.forward(ids)
    assert h.dtype == torch.float32 and torch.equal(h.cpu(), w["e"].float().cpu()[[3, 89, 0]])
    x = torch.randn(4, 24).to(dtype).to(DEV)
    logits = head.forward(x)
    assert logits.dtype == torch.float32
    assert rel_err(logits, x.double().cpu() @ w["e"].double().cpu().T) < (5e-6 if dtype == torch.float32 else 3e-3)


def shared_schedule_spec(H=48, V=70):
    """Two layers; the schedule runs layer 0, layer 1, layer 0 again (its own
    cache), then a third attention that has no k/v of its own and reads the
    cache of the first run."""
    from infernum_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleItem

    def layer(i, kv_shared=False):
        p = f"model.layers.{i}."
        norm = lambda n: PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5, "weight": p + n})  # noqa: E731
        return LayerSpec("prenorm", name=p, parts={
            "norm1": norm("n1"),
            "mixer": PartSpec("attention", {"hidden_size": H, "num_heads": 4, "num_kv_heads": 2,
                                            "head_dim": 16, "prefix": p + "attn.", "kv_shared": kv_shared,
                                            "position": {"kind": "rotary", "params": {"head_dim": 16, "theta": 1e4}}}),
            "norm2": norm("n2"),
            "ffn": PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 80, "prefix": p + "mlp."}),
        })

    return ModelSpec(
        hidden_size=H, vocab_size=V,
        embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "weight": "emb"}),
        layers=(layer(0), layer(1), layer(2, kv_shared=True)),
        schedule=(ScheduleItem(0), ScheduleItem(1), ScheduleItem(0), ScheduleItem(2, cache_of=0)),
        final_norm=PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5, "weight": "fn"}),
        lm_head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "weight": "head"}),
        max_position=256)


def plain_shared_schedule(W, tokens, H=48):
    T = len(tokens)
    W = {k: v.double().cpu() for k, v in W.items()}
    f = pl.rope_frequencies(16, 1e4, None)
    p = torch.arange(T)
    h = W["emb"][tokens]
    kept = {}
    for pos, (i, cache_of) in enumerate([(0, None), (1, None), (0, None), (2, 0)]):
        pre = f"model.layers.{i}."
        x = pl.rms_norm(h, W[pre + "n1"], 1e-5)
        q = pl.rope((x @ W[pre + "attn.q_proj.weight"].T).view(T, 4, 16), p, f)
        if cache_of is None:
            k = pl.rope((x @ W[pre + "attn.k_proj.weight"].T).view(T, 2, 16), p, f)
            v = (x @ W[pre + "attn.v_proj.weight"].T).view(T, 2, 16)
            kept[pos] = (k, v)
        else:
            k, v = kept[cache_of]
        h = h + pl.attention(q, k, v).reshape(T, 64) @ W[pre + "attn.o_proj.weight"].T
        m = pl.rms_norm(h, W[pre + "n2"], 1e-5)
        h = h + pl.swiglu(m, W[pre + "mlp.gate_proj.weight"], W[pre + "mlp.up_proj.weight"],
                          W[pre + "mlp.down_proj.weight"])
    return pl.rms_norm(h, W["fn"], 1e-5) @ W["head"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_schedule_names_a_layer_twice_and_shares_a_cache(dtype):
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry
    from infernum_b200.models.model import Model
    from infernum_b200.weights.random_init import random_tensors
    rt = runtime(dtype)
    model = Model(shared_schedule_spec(), rt)
    specs = model.weight_specs()
    assert "model.layers.2.attn.k_proj.weight" not in specs
    W = random_tensors(specs, 5, DEV, dtype)
    for k in W:
        if "proj" in k:
            W[k] = (W[k].float() * 6).to(dtype)
    model.bind(W)
    needs = model.cache_needs()
    assert [n.cache_of for n in needs] == [None, None, None, 0]
    cache = CacheManager(needs, page_size=4, num_pages=32, max_requests=2, dtype=dtype, device=DEV)
    assert len(cache.groups) == 1 and cache.groups[0].positions == [0, 1, 2]
    assert cache.layer_caches[3].k_pool is cache.layer_caches[0].k_pool
    assert cache.layer_caches[2].k_pool is not cache.layer_caches[0].k_pool
    runner = ModelRunner(model, cache)
    tokens = [int(t) for t in torch.randint(0, 70, (33,))]
    rc = cache.admit("a")
    rows, pos = [], 0
    for n in [9, 1, 2, 20, 1]:
        rows.append(runner.step([StepEntry(rc, tokens[pos: pos + n], list(range(n)))]))
        pos += n
    runner.check_errors()
    got = torch.cat(rows)
    assert rel_err(got, plain_shared_schedule(W, tokens)) < (2e-5 if dtype == torch.float32 else 4e-2)


def test_products_report_into_the_runtimes_error_word(monkeypatch):
    """The tensor-core products report a wait that ran out in the device word
    they are handed.  Every product of a part must be handed the word of the
    part's Runtime (the one the engine reads after a step), not one of their
    own: the calls are watched at the C boundary, for both kernels, with and
    without the activation in the epilogue."""
    from infernum_b200.ops import gemm_tc
    from infernum_b200.parts import FEED_FORWARDS
    from infernum_b200.parts.linear import Linear
    rt = runtime(torch.bfloat16)
    seen = {"few": [], "pair": []}
    few, pair = gemm_tc.lib(), gemm_tc.pair_lib()
    real_few, real_pair = few.ib_gemm_tc, pair.ib_gemm_pair

    def spy_few(*args):
        seen["few"].append(args[12])
        return real_few(*args)

    def spy_pair(*args):
        seen["pair"].append(args[15])
        return real_pair(*args)

    monkeypatch.setattr(few, "ib_gemm_tc", spy_few)
    monkeypatch.setattr(pair, "ib_gemm_pair", spy_pair)
    lin = Linear(torch.randn(160, 96, device=DEV).to(torch.bfloat16), rt)
    lin(torch.randn(5, 96, device=DEV).to(torch.bfloat16))          # few tokens
    lin(torch.randn(768, 96, device=DEV).to(torch.bfloat16))        # a prompt: pairs of SMs
    ffn = FEED_FORWARDS.get("swiglu")({"hidden_size": 96, "intermediate_size": 256, "prefix": "m."}, rt)
    ffn.bind(weights_for(ffn, torch.bfloat16))
    ffn.forward(torch.randn(3, 96, device=DEV).to(torch.bfloat16))    # activation in the epilogue, few tokens
    ffn.forward(torch.randn(512, 96, device=DEV).to(torch.bfloat16))  # and on pairs of SMs
    torch.cuda.synchronize()
    word = rt.err.data_ptr()
    assert len(seen["few"]) >= 3 and len(seen["pair"]) >= 2
    assert set(seen["few"]) == {word} and set(seen["pair"]) == {word}
    assert int(rt.err.item()) == 0


def test_random_weights_are_the_same_on_the_device_and_in_a_written_folder(tmp_path):
    """A model drawn on the GPU from a configuration and a seed and the folder
    written for the same configuration and seed hold the same values bit for
    bit, so what was measured on one can be checked with the plain
    implementation on the other."""
    from helpers import TINY_B
    from infernum_b200.weights.random_init import model_specs_for, random_tensors, write_random_model
    folder = write_random_model(str(tmp_path / "m"), TINY_B, seed=21)
    stored = pl.read_weights(folder)
    _, _, specs = model_specs_for(TINY_B)
    drawn = random_tensors(specs, 21, DEV, torch.bfloat16)
    assert set(stored) == set(drawn)
    for name, t in drawn.items():
        assert torch.equal(t.cpu(), stored[name]), name
    other = random_tensors(specs, 22, DEV, torch.bfloat16)
    assert not torch.equal(other["model.embed_tokens.weight"], drawn["model.embed_tokens.weight"])
