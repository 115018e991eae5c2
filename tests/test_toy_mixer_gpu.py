"""A toy mixer with state of its own, defined here, is registered, built and
stepped without a change to the package: the registries, the model
description, the cache manager's state slots and the step function carry it."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def define_toy():
    from infernum_b200.parts import (LayerSpec, Mixer, ModelSpec, PartSpec, ScheduleItem, StateSpec,
                                     WeightSpec, register_mixer)
    from infernum_b200.registry import register_architecture

    @register_mixer("toy_running_mean")
    class RunningMean(Mixer):
        """y_t = W . (decay * s_{t-1} + x_t), s carried per request in its state slot."""

        def __init__(self, params, rt):
            super().__init__(params, rt)
            self.h = params["hidden_size"]
            self.decay = params["decay"]
            self.name = params["prefix"] + "mix.weight"

        def state_spec(self):
            return StateSpec((self.h,), torch.float32)

        def weight_specs(self):
            return {self.name: WeightSpec((self.h, self.h))}

        def bind(self, weights):
            self.w = weights[self.name].float()

        def forward(self, x, ctx, cache):
            # What a mixer with state may rely on: how many rows and entries the step has is
            # known on the host and fixed for a recorded step; which row belongs to which entry
            # (``row_entry``) and which entry to which slot (``slot_ids``) is known on the device
            # only, because a recorded step is replayed for other requests, for portions of
            # other lengths, and with rows at its end that belong to no request (their entry's
            # slot is the spare one).  Nothing here reads device memory on the host, so the
            # engine can record it in a CUDA graph.
            state, xf = cache.state, x.float()
            if ctx.max_rows_per_entry == 1:  # one row per entry: all entries at once
                slots = ctx.slot_ids.long()
                s = state[slots] * self.decay + xf
                state[slots] = s  # (rows that pad a batch all write the spare slot)
                return (s @ self.w.T).to(x.dtype)
            out = torch.empty_like(x)
            slot_of_row = ctx.slot_ids.long()[ctx.row_entry.long()]
            for r in range(x.shape[0]):  # rows of a request come in order, its state is carried along
                slot = slot_of_row[r: r + 1]
                s = state[slot] * self.decay + xf[r: r + 1]
                state[slot] = s
                out[r: r + 1] = (s @ self.w.T).to(x.dtype)
            return out

    def build_spec(cfg):
        H, V = cfg["hidden_size"], cfg["vocab_size"]
        layers = []
        for i in range(cfg["num_hidden_layers"]):
            p = f"layers.{i}."
            norm = lambda n: PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5, "weight": p + n})  # noqa: E731
            mixer = PartSpec("toy_running_mean", {"hidden_size": H, "decay": cfg["decay"], "prefix": p}) \
                if i % 2 == 0 else PartSpec("attention", {
                    "hidden_size": H, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                    "prefix": p + "attn.", "window": cfg.get("window", 0) if i % 4 == 3 else 0,
                    "position": {"kind": "rotary", "params": {"head_dim": 16, "theta": 1e4}}})
            layers.append(LayerSpec("prenorm", name=p, parts={
                "norm1": norm("n1"), "mixer": mixer, "norm2": norm("n2"),
                "ffn": PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 2 * H, "prefix": p + "mlp."})}))
        return ModelSpec(
            hidden_size=H, vocab_size=V,
            embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "weight": "emb"}),
            layers=tuple(layers), schedule=tuple(ScheduleItem(i) for i in range(len(layers))),
            final_norm=PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5, "weight": "fn"}),
            lm_head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "weight": "head", "tied_to": "emb"}),
            max_position=128)

    register_architecture("toy-state", lambda d: dict(d), build_spec)


CFG = {"model_type": "toy-state", "hidden_size": 32, "vocab_size": 50, "num_hidden_layers": 3, "decay": 0.5}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_steps_like_a_whole_run(dtype, tmp_path):
    import infernum_b200 as ib
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry
    define_toy()
    # through a model folder, so the loader and the registry see the new architecture too
    folder = ib.write_random_model(str(tmp_path / "toy"), CFG, seed=3)
    model = ib.load_model(folder, dtype=dtype)
    needs = model.cache_needs()
    assert needs[0].state is not None and needs[0].paged is None and needs[1].paged is not None

    def run(cuts_a, cuts_b):
        cache = CacheManager(needs, page_size=4, num_pages=24, max_requests=3,
                             dtype=model.rt.dtype, device=DEV)
        # one row per request slot, and one more that rows padding a batch write to
        assert cache.layer_caches[0].state.shape == (3 + 1, 32) and cache.layer_caches[1].state is None
        runner = ModelRunner(model, cache)
        # a request that lived in the slot before leaves state behind: it must be zeroed
        old = cache.admit("old")
        runner.step([StepEntry(old, [1, 2, 3, 4, 5], [])])
        cache.release(old)
        seqs = {"a": [int(t) for t in torch.arange(30) % 50], "b": [int(t) for t in (torch.arange(17) * 7) % 50]}
        cuts = {"a": list(cuts_a), "b": list(cuts_b)}
        rcs = {k: cache.admit(k) for k in seqs}
        fed = {k: 0 for k in seqs}
        rows = {k: [] for k in seqs}
        while any(cuts.values()):
            entries, who = [], []
            for k in seqs:
                if cuts[k]:
                    n = cuts[k].pop(0)
                    entries.append(StepEntry(rcs[k], seqs[k][fed[k]: fed[k] + n], list(range(n))))
                    fed[k] += n
                    who.append((k, n))
            logits = runner.step(entries)
            off = 0
            for k, n in who:
                rows[k].append(logits[off: off + n])
                off += n
        runner.check_errors()
        assert fed == {"a": 30, "b": 17}
        return {k: torch.cat(v).cpu() for k, v in rows.items()}

    whole = run([30], [17])
    cut = run([7, 1, 2, 13, 1, 6], [2, 9, 1, 1, 4])
    tol = 1e-5 if dtype == "float32" else 3e-2
    for k in whole:
        assert torch.isfinite(whole[k]).all()
        scale = whole[k].abs().max()
        assert (whole[k] - cut[k]).abs().max() / scale < tol
    assert (whole["a"][:17] - whole["b"]).abs().max() > 1e-3  # the two requests are not mixed up


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_through_the_engine(dtype, tmp_path):
    """The same toy architecture through ``Engine`` as a user runs it: decode
    steps recorded as CUDA graphs and launched ahead, rows that pad a batch, a
    request that arrives late, and page pools so small that a request is
    preempted, loses its state slot and is computed again.  Four layers: state,
    attention over all keys, state, attention with a window - so the cache has
    two groups of pages, sized apart, beside the state slots.  Every request
    gets the tokens of its run alone, and those are the tokens of one whole
    pass over prompt and continuation."""
    import infernum_b200 as ib
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry
    define_toy()
    cfg = dict(CFG, num_hidden_layers=4, window=12)
    folder = ib.write_random_model(str(tmp_path / "toy4"), cfg, seed=5)
    model = ib.load_model(folder, dtype=dtype)
    needs = model.cache_needs()
    assert [n.paged.window if n.paged else None for n in needs] == [None, 0, None, 12]
    prompts = [[(7 * i + 3 * j) % 50 for j in range(n)] for i, n in enumerate((9, 21, 5, 14))]
    n_new = 30
    opts = ib.GenerateOptions(max_new_tokens=n_new, ignore_eos=True)
    base = dict(max_batch_size=4, block_size=4, max_prefill_tokens=8, max_model_len=64)
    solo = ib.Engine(model, ib.BatchConfig(num_blocks=[16, 16], cuda_graphs=False, **base))
    alone = [solo.generate(p, opts) for p in prompts]
    # the pool of the group that keeps every key holds 30 pages where the four requests need 43;
    # the windowed group gets by with pages_for(12 + 8) + 1 = 6 a request
    tight = ib.Engine(model, ib.BatchConfig(num_blocks=[30, 24], **base))
    assert tight.cache.group_pages == [30, 24] and tight.decoder is not None
    handles = [tight.submit(p, opts) for p in prompts[:3]]
    for _ in range(6):
        tight.step()
    handles.append(tight.submit(prompts[3], opts))  # arrives while the others decode
    tight.run_until_done(handles)
    assert tight.stats.preemptions > 0 and tight.stats.ahead_launched > 0
    assert any(s.graph is not None for s in tight.decoder._slots.values())
    assert tight.cache.free_pages() == [30, 24] and tight.cache.num_free_slots == 4
    for h, want in zip(handles, alone):
        assert len(h.tokens) == n_new
        if dtype == "float32":
            assert h.tokens == want
    if dtype == "float32":
        # one whole pass over prompt and continuation selects the same tokens
        cache = CacheManager(needs, page_size=4, num_pages=[16, 16], max_requests=1, dtype=model.rt.dtype, device=DEV)
        runner = ModelRunner(model, cache)
        for p, want in zip(prompts, alone):
            rc = cache.admit("whole")
            seq = p + want[:-1]
            logits = runner.step([StepEntry(rc, seq, list(range(len(p) - 1, len(seq))))])
            assert logits.argmax(dim=1).tolist() == want
            cache.release(rc)
        runner.check_errors()


def define_toy_parts():
    """A position encoding and a routed feed-forward defined here, registered
    through the package's registries."""
    from infernum_b200.parts import (FeedForward, PositionEncoding, WeightSpec, register_feed_forward,
                                     register_position_encoding)

    @register_position_encoding("toy_scaled")
    class ScaledPositions(PositionEncoding):
        """q and k are scaled by (1 + rate * position): not a rotation, so the
        attention part must take its general route (apply, then store k and v)."""

        def __init__(self, params, rt):
            super().__init__(params, rt)
            self.rate = params["rate"]

        def apply(self, q, k, positions):
            f = (1.0 + self.rate * positions.float()).to(q.dtype)
            q.mul_(f[:, None, None])
            if k is not None:
                k.mul_(f[:, None, None])

    @register_feed_forward("toy_routed")
    class RoutedFFN(FeedForward):
        """Each token goes to the expert with the largest router logit (computed
        in 32-bit); an expert is one matrix.  It asks the device which rows chose
        which expert, so it cannot be replayed from a recording and says so."""

        replayable = False

        def __init__(self, params, rt):
            super().__init__(params, rt)
            self.h, self.n, self.prefix = params["hidden_size"], params["experts"], params["prefix"]

        def weight_specs(self):
            specs = {self.prefix + "router.weight": WeightSpec((self.n, self.h), std=1.0)}
            for i in range(self.n):
                specs[self.prefix + f"experts.{i}.weight"] = WeightSpec((self.h, self.h), std=0.1)
            return specs

        def bind(self, weights):
            self.router = weights[self.prefix + "router.weight"].float()
            self.experts = [weights[self.prefix + f"experts.{i}.weight"] for i in range(self.n)]

        def forward(self, x, ctx):
            choice = (x.float() @ self.router.T).argmax(dim=-1)
            out = torch.zeros_like(x)
            for i, w in enumerate(self.experts):
                rows = (choice == i).nonzero().flatten()
                if rows.numel():
                    out[rows] = (x[rows].float() @ w.float().T).to(x.dtype)
            return out


def toy_parts_spec(H=48, V=60):
    from infernum_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleItem
    layers = []
    for i in range(2):
        p = f"layers.{i}."
        norm = lambda n: PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5, "weight": p + n})  # noqa: E731
        layers.append(LayerSpec("prenorm", name=p, parts={
            "norm1": norm("n1"),
            "mixer": PartSpec("attention", {"hidden_size": H, "num_heads": 3, "num_kv_heads": 3, "head_dim": 16,
                                            "prefix": p + "attn.",
                                            "position": {"kind": "toy_scaled", "params": {"rate": 0.02}}}),
            "norm2": norm("n2"),
            "ffn": PartSpec("toy_routed", {"hidden_size": H, "experts": 3, "prefix": p + "moe."}) if i == 1
            else PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 96, "prefix": p + "mlp."})}))
    return ModelSpec(
        hidden_size=H, vocab_size=V,
        embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "weight": "emb"}),
        layers=tuple(layers), schedule=(ScheduleItem(0), ScheduleItem(1)),
        final_norm=PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5, "weight": "fn"}),
        lm_head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "weight": "head"}), max_position=128)


def test_toy_position_encoding_and_routed_feed_forward():
    """Different feed-forwards in different layers, a position encoding the
    attention part has no fused route for: whole prompts equal portions, and
    the first layer equals a by-hand float64 computation."""
    import plain_llama as pl
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry
    from infernum_b200.models.model import Model
    from infernum_b200.ops import core
    from infernum_b200.parts.base import Runtime
    from infernum_b200.weights.random_init import random_tensors
    define_toy_parts()
    rt = Runtime(DEV, torch.float32, err=core.new_error_word(DEV))
    model = Model(toy_parts_spec(), rt)
    W = random_tensors(model.weight_specs(), 9, DEV, torch.float32)
    for k in W:
        if "attn" in k:
            W[k] = W[k] * 8
    model.bind(W)
    tokens = [int(t) for t in (torch.arange(37) * 11) % 60]

    def run(cuts):
        cache = CacheManager(model.cache_needs(), page_size=4, num_pages=16, max_requests=1,
                             dtype=torch.float32, device=DEV)
        runner = ModelRunner(model, cache)
        rc = cache.admit("r")
        rows, pos = [], 0
        for n in cuts:
            rows.append(runner.step([StepEntry(rc, tokens[pos: pos + n], list(range(n)))]))
            pos += n
        runner.check_errors()
        return torch.cat(rows).cpu()

    whole, cut = run([37]), run([5, 1, 9, 2, 1, 19])
    assert torch.isfinite(whole).all()
    assert (whole - cut).abs().max() / whole.abs().max() < 1e-5
    # layer 0's attention by hand: scaled q and k instead of rotated ones
    Wd = {k: v.double().cpu() for k, v in W.items()}
    T = len(tokens)
    h = Wd["emb"][tokens]
    x = pl.rms_norm(h, Wd["layers.0.n1"], 1e-5)
    f = (1.0 + 0.02 * torch.arange(T, dtype=torch.float32)).double()[:, None, None]
    q = (x @ Wd["layers.0.attn.q_proj.weight"].T).view(T, 3, 16) * f
    k = (x @ Wd["layers.0.attn.k_proj.weight"].T).view(T, 3, 16) * f
    v = (x @ Wd["layers.0.attn.v_proj.weight"].T).view(T, 3, 16)
    h = h + pl.attention(q, k, v).reshape(T, 48) @ Wd["layers.0.attn.o_proj.weight"].T
    h = h + pl.swiglu(pl.rms_norm(h, Wd["layers.0.n2"], 1e-5), Wd["layers.0.mlp.gate_proj.weight"],
                      Wd["layers.0.mlp.up_proj.weight"], Wd["layers.0.mlp.down_proj.weight"])
    # layer 1: attention the same way, then the routed feed-forward
    x = pl.rms_norm(h, Wd["layers.1.n1"], 1e-5)
    q = (x @ Wd["layers.1.attn.q_proj.weight"].T).view(T, 3, 16) * f
    k = (x @ Wd["layers.1.attn.k_proj.weight"].T).view(T, 3, 16) * f
    v = (x @ Wd["layers.1.attn.v_proj.weight"].T).view(T, 3, 16)
    h = h + pl.attention(q, k, v).reshape(T, 48) @ Wd["layers.1.attn.o_proj.weight"].T
    m = pl.rms_norm(h, Wd["layers.1.n2"], 1e-5)
    choice = (m @ Wd["layers.1.moe.router.weight"].T).argmax(dim=-1)
    moe = torch.stack([m[t] @ Wd[f"layers.1.moe.experts.{int(choice[t])}.weight"].T for t in range(T)])
    h = h + moe
    want = pl.rms_norm(h, Wd["fn"], 1e-5) @ Wd["head"].T
    assert (whole.double() - want).abs().max() / want.abs().max() < 5e-5
    assert len(set(choice.tolist())) > 1  # more than one expert was used


def test_a_part_that_cannot_be_replayed_keeps_the_engine_eager():
    """The routed feed-forward above reads its routing back on the host, so
    it declares ``replayable = False``: an engine with it records no step and
    still generates what one whole pass selects."""
    import infernum_b200 as ib
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry
    from infernum_b200.models.model import Model
    from infernum_b200.ops import core
    from infernum_b200.parts.base import Runtime
    from infernum_b200.weights.random_init import random_tensors
    define_toy_parts()
    rt = Runtime(DEV, torch.float32, err=core.new_error_word(DEV))
    model = Model(toy_parts_spec(), rt)
    model.bind(random_tensors(model.weight_specs(), 4, DEV, torch.float32))
    assert not model.replayable and model.layers[0].all_replayable() and not model.layers[1].all_replayable()
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=2, block_size=4, num_blocks=32, max_model_len=64))
    assert engine.decoder is None
    prompt = [3, 14, 15, 9, 2, 6]
    got = engine.generate(prompt, ib.GenerateOptions(max_new_tokens=12, ignore_eos=True))
    cache = CacheManager(model.cache_needs(), page_size=4, num_pages=16, max_requests=1, dtype=torch.float32, device=DEV)
    rc = cache.admit("whole")
    seq = prompt + got[:-1]
    logits = ModelRunner(model, cache).step([StepEntry(rc, seq, list(range(len(prompt) - 1, len(seq))))])
    assert logits.argmax(dim=1).tolist() == got
