"""Generation through the Python entry point and the command line: greedy
tokens equal the plain implementation's; batched equals alone; sampling is
reproducible and independent of the batch; preemption leaves output unchanged."""
import os
import subprocess
import sys

import pytest
import torch

import plain_llama as pl
from helpers import CONFIGS, ROOT, Plain, assert_same_up_to_ties, make_model_folder, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    # sharpened models: logit gaps are far above bfloat16 noise, so greedy tokens are stable
    return {n: make_model_folder(str(tmp_path_factory.mktemp(f"gen{n}")), CONFIGS[n], 60 + i, sharpen=6.0)
            for i, n in enumerate(["A", "B"])}


def plain_greedy_with_margin(folder, prompt, n):
    """Greedy tokens of the plain implementation and the smallest gap between
    the best and second-best logit along the way (relative to the largest)."""
    cfg, w = pl.read_config(folder), pl.read_weights(folder)
    seq, out, margin = list(prompt), [], 1e9
    for _ in range(n):
        logits = pl.forward(cfg, w, seq)[-1]
        top = torch.topk(logits, 2).values
        margin = min(margin, float((top[0] - top[1]) / logits.abs().max()))
        t = pl.argmax(logits)
        out.append(t)
        seq.append(t)
    return out, margin


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_equals_plain(folders, name, dtype):
    import infernum_b200 as ib
    model = ib.load_model(folders[name], dtype=dtype)
    block = {"A": 4, "B": 8}[name]
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=4, max_prefill_tokens=7, block_size=block,
                                             num_blocks=64, max_tokens_per_step=16))
    vocab = CONFIGS[name]["vocab_size"]
    lens = {"A": [5, 17, 33], "B": [1, 9, 40]}[name]
    prompts = [random_tokens(n, vocab, 7 * n) for n in lens]
    n_new = {"A": 16, "B": 24}[name]
    opts = ib.GenerateOptions(max_new_tokens=n_new)
    got_batch = engine.generate_batch(prompts, opts)
    plain = Plain(folders[name])
    compared = 0
    for p, got in zip(prompts, got_batch):
        want, _ = plain_greedy_with_margin(folders[name], p, n_new)
        # token for token, up to the first step at which the engine took another token; that
        # step must be a near-tie by the plain logits (within the dtype's noise)
        compared += assert_same_up_to_ties(plain, p, got, want, dtype)
        assert engine.generate(p, opts) == got  # alone equals batched
    assert compared >= (len(prompts) * n_new if dtype == "float32" else n_new)
    assert engine.cache.free_pages() == [64] and engine.cache.num_free_slots == 4


def test_stream_eos_and_length(folders):
    import infernum_b200 as ib
    model = ib.load_model(folders["A"], dtype="float32")
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=2, block_size=4, num_blocks=64))
    prompt = random_tokens(9, 256, 1)
    full = engine.generate(prompt, ib.GenerateOptions(max_new_tokens=12))
    assert list(engine.generate_stream(prompt, ib.GenerateOptions(max_new_tokens=12))) == full
    stop = full[5]
    first = full.index(stop)
    cut = engine.generate(prompt, ib.GenerateOptions(max_new_tokens=12, eos_token_id=stop))
    assert cut == full[:first]  # the end-of-sequence token is neither kept nor emitted
    h = engine.submit(prompt, ib.GenerateOptions(max_new_tokens=12, eos_token_id=stop))
    engine.run_until_done([h])
    assert h.finish_reason == ib.FinishReason.STOP and h.events[-1].kind == "finished"
    with pytest.raises(ib.InfernumError):
        engine.submit([1, 2, 999], ib.GenerateOptions())
    with pytest.raises(ib.SchedulingError):
        engine.submit([1] * 120, ib.GenerateOptions(max_new_tokens=20))


def test_sampling_is_seeded_and_independent_of_the_batch(folders):
    import infernum_b200 as ib
    model = ib.load_model(folders["B"], dtype="float32")
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=4, block_size=8, num_blocks=64,
                                             max_prefill_tokens=16, max_tokens_per_step=24))
    prompts = [random_tokens(n, 320, n) for n in (6, 21, 40)]
    opts = [ib.GenerateOptions(max_new_tokens=20, sampling=ib.SamplingParams(
        temperature=0.8, top_p=0.9, seed=100 + i, repetition_penalty=1.2)) for i in range(3)]
    together = engine.generate_batch(prompts, opts)
    again = engine.generate_batch(prompts, opts)
    assert together == again
    for p, o, t in zip(prompts, opts, together):
        assert engine.generate(p, o) == t
    other = engine.generate(prompts[1], ib.GenerateOptions(max_new_tokens=20, sampling=ib.SamplingParams(
        temperature=0.8, top_p=0.9, seed=999, repetition_penalty=1.2)))
    assert other != together[1]
    greedy = engine.generate(prompts[1], ib.GenerateOptions(max_new_tokens=20))
    assert greedy != together[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_leaves_output_unchanged(folders, dtype):
    import infernum_b200 as ib
    model = ib.load_model(folders["A"], dtype=dtype)
    prompts = [random_tokens(9, 256, 50 + i) for i in range(3)]
    opts = [ib.GenerateOptions(max_new_tokens=40),
            ib.GenerateOptions(max_new_tokens=40, sampling=ib.SamplingParams(temperature=0.7, seed=5)),
            ib.GenerateOptions(max_new_tokens=40)]
    roomy = ib.Engine(model, ib.BatchConfig(max_batch_size=3, block_size=4, num_blocks=64))
    want = [roomy.generate(p, o) for p, o in zip(prompts, opts)]
    tight = ib.Engine(model, ib.BatchConfig(max_batch_size=3, block_size=4, num_blocks=24,
                                            max_prefill_tokens=8))
    got = tight.generate_batch(prompts, opts)
    assert tight.stats.preemptions > 0
    for p, o, g, w in zip(prompts, opts, got, want):
        assert_same_up_to_ties(folders["A"], p, g, w, dtype, sampling=o.sampling)
    assert tight.cache.free_pages() == [24]


def test_command_line_generate(folders):
    env = dict(os.environ, LLAMA_MODEL_PATH=folders["A"])
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "5,6,7,8", "-n", "6",
                          "--greedy", "--dtype", "float32", "--block-size", "4"],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    assert "Decoding: greedy (argmax)" in out.stdout and "Generated 6 tokens" in out.stdout
    line = [l for l in out.stdout.splitlines() if l.startswith("5,6,7,8")][0]
    got = [int(t) for t in line.split()[1:]]
    want, _ = plain_greedy_with_margin(folders["A"], [5, 6, 7, 8], 6)
    assert got == want
    out2 = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "-m", folders["A"],
                           "5,6,7,8", "-n", "5", "-t", "0.9", "-p", "0.8", "-s", "7", "-r", "1.3",
                           "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert out2.returncode == 0, out2.stderr[-3000:]
    assert "Sampling: temperature=0.9, top_p=0.8, seed=7, repetition_penalty=1.3 (window=64)" in out2.stdout


def test_command_line_generate_from_a_bare_configuration(tmp_path):
    """``--config FILE --random-weights``: from a config.json and a seed to tokens
    with no checkpoint; the weights are those ``write_random_model`` writes for the
    same two, so the plain implementation can check the tokens."""
    import json
    from infernum_b200.weights.random_init import write_random_model
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CONFIGS["B"]))
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "--config", str(cfg_path),
                          "--random-weights", "--weights-seed", "9", "5,6,7,8,9", "-n", "5", "--greedy",
                          "--dtype", "float32", "--block-size", "8"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("5,6,7,8,9")][0]
    got = [int(t) for t in line.split()[1:]]
    folder = write_random_model(str(tmp_path / "same"), CONFIGS["B"], 9)
    want, _ = plain_greedy_with_margin(folder, [5, 6, 7, 8, 9], 5)
    assert_same_up_to_ties(folder, [5, 6, 7, 8, 9], got, want, "float32")
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "--random-weights", "1,2"],
                         capture_output=True, text=True, timeout=600)
    assert bad.returncode == 2 and "go together" in bad.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_come_and_go_under_recorded_decode_graphs(folders, dtype):
    """Requests of different lengths leave the batch one by one and a late one
    joins: the decode graphs are recorded per batch bucket, not per set of
    requests, rows that only pad a bucket do no harm, and every request gets
    the tokens it gets alone."""
    import infernum_b200 as ib
    model = ib.load_model(folders["B"], dtype=dtype)
    cfg = ib.BatchConfig(max_batch_size=8, block_size=8, num_blocks=96, max_prefill_tokens=64)
    engine = ib.Engine(model, cfg)
    prompts = [random_tokens(n, 320, 30 + n) for n in (3, 11, 7, 20, 5)]
    news = [4, 30, 9, 17, 24]
    opts = [ib.GenerateOptions(max_new_tokens=n) for n in news]
    handles = [engine.submit(p, o) for p, o in zip(prompts[:4], opts[:4])]
    for _ in range(6):
        engine.step()
    handles.append(engine.submit(prompts[4], opts[4]))  # joins while the others decode
    engine.run_until_done(handles)
    recorded = [k for k, s in engine.decoder._slots.items() if s.graph is not None]
    assert recorded and len(recorded) <= 4  # buckets 1, 2, 4, 8 at most: not one per composition
    solo = ib.Engine(model, cfg)
    for p, o, h in zip(prompts, opts, handles):
        assert len(h.tokens) == o.max_new_tokens
        assert_same_up_to_ties(folders["B"], p, h.tokens, solo.generate(p, o), dtype)
    assert engine.cache.free_pages() == [96] and engine.cache.num_free_slots == 8


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_planned_ahead_survive_ends_and_arrivals(folders, dtype):
    """With launching ahead switched off: while a step runs, the engine plans the
    next one and keeps the plan until the tokens have come.  A request that ends
    on an end-of-sequence token and one that is cancelled void such a plan, one
    that arrives joins a step later; the tokens of the others do not change."""
    import infernum_b200 as ib
    model = ib.load_model(folders["B"], dtype=dtype)
    cfg = ib.BatchConfig(max_batch_size=4, block_size=8, num_blocks=96, max_prefill_tokens=64, launch_ahead=False)
    solo = ib.Engine(model, cfg)
    prompts = [random_tokens(n, 320, 70 + n) for n in (5, 9, 14, 6)]
    sampled = ib.SamplingParams(temperature=0.9, top_p=0.95, seed=3, repetition_penalty=1.3)
    alone = [solo.generate(prompts[0], ib.GenerateOptions(max_new_tokens=30)),
             solo.generate(prompts[1], ib.GenerateOptions(max_new_tokens=30, sampling=sampled)),
             solo.generate(prompts[2], ib.GenerateOptions(max_new_tokens=30)),
             solo.generate(prompts[3], ib.GenerateOptions(max_new_tokens=12))]
    stop = alone[0][10]  # request 0 ends where this token first shows
    engine = ib.Engine(model, cfg)
    h0 = engine.submit(prompts[0], ib.GenerateOptions(max_new_tokens=30, eos_token_id=stop))
    h1 = engine.submit(prompts[1], ib.GenerateOptions(max_new_tokens=30, sampling=sampled))
    h2 = engine.submit(prompts[2], ib.GenerateOptions(max_new_tokens=30))
    for _ in range(5):
        engine.step()
    h3 = engine.submit(prompts[3], ib.GenerateOptions(max_new_tokens=12))  # arrives
    while len(h2.tokens) < 20:
        engine.step()
    engine.cancel(h2)
    engine.run_until_done([h0, h1, h3])
    assert engine.stats.ahead_used > 10 and engine.stats.ahead_voided >= 2 and engine.stats.ahead_launched == 0
    assert h3.finish_reason == ib.FinishReason.LENGTH and len(h3.tokens) == 12 and len(h1.tokens) == 30
    # token for token; in bfloat16 the solo engine may round a near-tie otherwise, and what comes
    # after such a step is not compared
    plain = Plain(folders["B"])
    assert_same_up_to_ties(plain, prompts[0], h0.tokens, alone[0][: len(h0.tokens)], dtype)
    if dtype == "float32":
        assert h0.tokens == alone[0][: alone[0].index(stop)] and h0.finish_reason == ib.FinishReason.STOP
    assert_same_up_to_ties(plain, prompts[1], h1.tokens, alone[1], dtype, sampling=sampled)
    assert_same_up_to_ties(plain, prompts[2], h2.tokens, alone[2][: len(h2.tokens)], dtype)
    assert_same_up_to_ties(plain, prompts[3], h3.tokens, alone[3], dtype)
    engine.step()
    assert engine.cache.free_pages() == [96] and engine.cache.num_free_slots == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_launched_ahead_of_their_tokens(folders, dtype):
    """The next decode step is launched behind the one in flight, fed on the device,
    before the host has read that one's tokens.  A request that then turns out to
    have ended (end-of-sequence, cancel) drops the token computed in vain, one that
    arrives joins a step later; nobody's tokens change against an engine that
    launches every step after reading the one before, greedy or sampled."""
    import infernum_b200 as ib
    model = ib.load_model(folders["B"], dtype=dtype)
    prompts = [random_tokens(n, 320, 170 + n) for n in (5, 9, 14, 6)]
    sampled = ib.SamplingParams(temperature=0.9, top_p=0.95, seed=3)  # no penalty: nothing to wait for
    base = dict(max_batch_size=4, block_size=8, num_blocks=96, max_prefill_tokens=64)
    solo = ib.Engine(model, ib.BatchConfig(launch_ahead=False, **base))
    stop = solo.generate(prompts[0], ib.GenerateOptions(max_new_tokens=30))[10]

    def run(ahead):
        engine = ib.Engine(model, ib.BatchConfig(launch_ahead=ahead, **base))
        h0 = engine.submit(prompts[0], ib.GenerateOptions(max_new_tokens=30, eos_token_id=stop))
        h1 = engine.submit(prompts[1], ib.GenerateOptions(max_new_tokens=40, sampling=sampled))
        h2 = engine.submit(prompts[2], ib.GenerateOptions(max_new_tokens=40))
        for _ in range(5):
            engine.step()
        h3 = engine.submit(prompts[3], ib.GenerateOptions(max_new_tokens=12))  # arrives
        while len(h2.tokens) < 20:
            engine.step()
        engine.cancel(h2)
        engine.run_until_done([h0, h1, h3])
        while engine.has_work():
            engine.step()
        assert engine.cache.free_pages() == [96] and engine.cache.num_free_slots == 4
        assert engine.decoder is None or not engine.decoder._reads  # every launched step was read
        return [h.tokens for h in (h0, h1, h2, h3)], [h.finish_reason for h in (h0, h1, h2, h3)], engine.stats

    on, on_reasons, on_stats = run(True)
    off, off_reasons, off_stats = run(False)
    assert on_stats.ahead_launched > 20 and off_stats.ahead_launched == 0
    assert on_reasons == off_reasons == [ib.FinishReason.STOP, ib.FinishReason.LENGTH,
                                         ib.FinishReason.CANCELLED, ib.FinishReason.LENGTH]
    if dtype == "float32":  # token for token
        assert on == off
    plain = Plain(folders["B"])  # in bfloat16 a near-tie may round otherwise in another batch
    for k, samp in enumerate([None, sampled, None, None]):
        n = min(len(on[k]), len(off[k]))  # (a request that was cancelled or stopped may have ended a token apart)
        assert_same_up_to_ties(plain, prompts[k], on[k][:n], off[k][:n], dtype, sampling=samp)


def test_stream_that_ends_on_a_stop_token_leaves_no_step_behind(folders):
    """A streamed request that ends on its end-of-sequence token has a step in
    flight that was launched ahead; it is read and dropped before the call
    returns, and the next request starts from a clean engine."""
    import infernum_b200 as ib
    model = ib.load_model(folders["B"], dtype="float32")
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=2, block_size=8, num_blocks=32))
    prompt = random_tokens(9, 320, 411)
    whole = engine.generate(prompt, ib.GenerateOptions(max_new_tokens=24))
    stop = whole[12]
    got = list(engine.generate_stream(prompt, ib.GenerateOptions(max_new_tokens=24, eos_token_id=stop)))
    assert got == whole[: whole.index(stop)]
    assert engine.stats.ahead_launched > 0
    assert (engine._ahead is None or not engine._ahead[2]) and not engine.decoder._reads
    assert engine.cache.free_pages() == [32] and engine.cache.num_free_slots == 2
    assert engine.generate(prompt, ib.GenerateOptions(max_new_tokens=24)) == whole


def test_self_feeding_decode_steps_with_and_without_graph_equal_the_engine(folders):
    """Decode steps that feed themselves on the device (the selected token and the
    advanced position of one step are the input of the next, with no copy from
    the host between them) launched kernel by kernel, the same replayed from a
    graph, and the engine's host-fed steps give the same tokens.  Kernels start
    under their predecessor's tail and read positions early: the step before
    must be complete by then."""
    import infernum_b200 as ib
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.decode import DecodeRunner
    from infernum_b200.engine.step import ModelRunner, StepEntry
    from infernum_b200.ops import core
    model = ib.load_model(folders["B"], dtype="float32")
    prompts = [random_tokens(n, 320, 90 + n) for n in (7, 30, 12)]
    steps = 40
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=4, block_size=8, num_blocks=96))
    want = engine.generate_batch(prompts, ib.GenerateOptions(max_new_tokens=steps + 1))
    for use_graph in (False, True):
        cache = CacheManager(model.cache_needs(), page_size=8, num_pages=96, max_requests=4,
                             dtype=model.rt.dtype, device=model.rt.device)
        runner = ModelRunner(model, cache, max_rows=64, max_entries=4)
        caches, first = [], []
        for i, p in enumerate(prompts):
            rc = cache.admit(("r", i))
            logits = runner.step([StepEntry(rc, p, [len(p) - 1])])
            out = torch.empty(1, dtype=torch.int32, device=logits.device)
            core.argmax(logits, out)
            caches.append(rc)
            first.append(int(out.item()))
        assert first == [w[0] for w in want]
        session = DecodeRunner(runner, 128, use_graph=use_graph)
        session.pin(caches, first, steps)
        # nothing is launched between the steps; a token or position read too early
        # in any of them changes what the last one selects
        for _ in range(steps):
            last = session.step_pinned()
        torch.cuda.synchronize()
        runner.check_errors()
        assert last.tolist() == [w[steps] for w in want], f"use_graph={use_graph}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_decoded_tokens_beside_one_prompt_portion_run_from_graphs(folders, dtype):
    """While a long prompt is fed in portions beside requests that decode, the
    steps recur with the same shape (a batch bucket of decoded tokens, then one
    portion): they are recorded as graphs like steps of decoded tokens alone.
    Every request gets the tokens it gets alone."""
    import infernum_b200 as ib
    model = ib.load_model(folders["B"], dtype=dtype)
    cfg = ib.BatchConfig(max_batch_size=8, block_size=8, num_blocks=128, max_prefill_tokens=64,
                         max_tokens_per_step=80)
    solo = ib.Engine(model, cfg)
    short = [random_tokens(n, 320, 200 + n) for n in (5, 9, 3)]
    long = random_tokens(230, 320, 77)
    sampled = ib.SamplingParams(temperature=0.8, top_p=0.9, seed=11)
    opts = [ib.GenerateOptions(max_new_tokens=40), ib.GenerateOptions(max_new_tokens=40, sampling=sampled),
            ib.GenerateOptions(max_new_tokens=40)]
    long_opts = ib.GenerateOptions(max_new_tokens=12)
    alone = [solo.generate(p, o) for p, o in zip(short, opts)] + [solo.generate(long, long_opts)]
    engine = ib.Engine(model, cfg)
    handles = [engine.submit(p, o) for p, o in zip(short, opts)]
    for _ in range(4):
        engine.step()
    handles.append(engine.submit(long, long_opts))  # fed 64 tokens at a time beside three decoding requests
    engine.run_until_done(handles)
    mixed = [k for k, s in engine.decoder._slots.items() if k[4] > 0]
    # recorded per bucket of the portions' rows: 64 for the full portions, 48 for the last 38 tokens
    # of the long prompt, 32 for the three short prompts, which came together (17 rows)
    assert mixed and {k[4] for k in mixed} <= {32, 48, 64}
    assert any(engine.decoder._slots[k].graph is not None for k in mixed)
    plain = Plain(folders["B"])
    for p, h, want in zip(short + [long], handles, alone):
        assert_same_up_to_ties(plain, p, h.tokens, want, dtype, sampling=h.seq.options.sampling)
    assert engine.cache.free_pages() == [128]


def test_a_request_admitted_again_does_not_inherit_its_old_block_table(folders):
    """The decode runner mirrors block tables row by row and refreshes only what
    changed.  A request that was released (preempted) and admitted again under
    the same id holds other pages, possibly as many as before: its row must be
    rewritten, or the step would read the pages it used to own."""
    import infernum_b200 as ib
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.decode import DecodeRunner
    from infernum_b200.engine.step import ModelRunner, StepEntry
    model = ib.load_model(folders["B"], dtype="float32")
    cfg, weights = pl.read_config(folders["B"]), pl.read_weights(folders["B"])
    cache = CacheManager(model.cache_needs(), page_size=8, num_pages=32, max_requests=4,
                         dtype=model.rt.dtype, device=model.rt.device)
    runner = ModelRunner(model, cache, max_rows=64, max_entries=4)
    session = DecodeRunner(runner, 64, use_graph=True)
    seq = random_tokens(22, 320, 5)

    def prefill_and_decode(rc):
        runner.step([StepEntry(rc, seq[:20], [])])
        cache.extend(rc, 1)
        session.step([rc], [seq[20]])
        logits = session.last.logits[0].float().cpu()
        want = pl.forward(cfg, weights, seq[:21])[-1]
        assert float((logits - want).abs().max() / want.abs().max()) < 2e-5

    first = cache.admit("a")
    prefill_and_decode(first)
    old_pages = list(first.tables[0])
    cache.release(first)
    squatter = cache.admit("x")          # takes the pages that were just given back
    cache.extend(squatter, 8 * len(old_pages))
    runner.step([StepEntry(squatter, random_tokens(8 * len(old_pages), 320, 6), [])])
    again = cache.admit("a")             # the same id, other pages, the same number of them
    prefill_and_decode(again)
    assert len(again.tables[0]) == len(old_pages) and set(again.tables[0]).isdisjoint(old_pages)


def test_a_product_whose_wait_ran_out_surfaces_from_engine_step(folders):
    """The engine reads one device word after every step.  A bit that a matrix
    product sets there (here set from the host: no kernel has to misbehave)
    ends the step with a KernelError that names the product and the wait."""
    import infernum_b200 as ib
    from infernum_b200.ops import core
    for graphs in (True, False):
        model = ib.load_model(folders["B"], dtype="bfloat16")
        engine = ib.Engine(model, ib.BatchConfig(max_batch_size=2, block_size=8, num_blocks=32, cuda_graphs=graphs))
        prompt = random_tokens(9, 320, 3)
        engine.generate(prompt, ib.GenerateOptions(max_new_tokens=4))  # graphs recorded, nothing reported
        site = core.TIMEOUT_SITES.index("product for few tokens: MMA issuer")
        engine.submit(prompt, ib.GenerateOptions(max_new_tokens=8))
        engine.step()
        model.rt.err.fill_(core.FLAG_WAIT_TIMEOUT | (1 << (8 + site)))
        with pytest.raises(ib.KernelError, match="product for few tokens: MMA issuer"):
            for _ in range(4):
                engine.step()
        assert int(model.rt.err.item()) == 0  # reported once, then cleared


def test_a_long_repetition_window_is_seen_whole_by_recorded_steps(folders):
    """The recent tokens of a sampling row sit in a buffer of fixed width in a
    recorded decode step.  A window longer than that buffer's smallest size (64)
    must still be seen whole: an engine that records its steps and one that
    launches them kernel by kernel select the same tokens, and the penalty over
    tokens 65 to 100 back does change them."""
    import infernum_b200 as ib
    model = ib.load_model(folders["B"], dtype="float32")
    prompt = random_tokens(20, 320, 808)
    base = dict(max_batch_size=2, block_size=8, num_blocks=64)

    def run(graphs, window):
        engine = ib.Engine(model, ib.BatchConfig(cuda_graphs=graphs, **base))
        sp = ib.SamplingParams(temperature=0.9, top_p=0.95, seed=4, repetition_penalty=1.8,
                               repetition_penalty_window=window)
        # a greedy request rides along, so that the batch has rows of both kinds
        out = engine.generate_batch([prompt, prompt[:7]], [ib.GenerateOptions(max_new_tokens=150, sampling=sp),
                                                           ib.GenerateOptions(max_new_tokens=150)])
        return out, engine

    (eager, eager_greedy), _ = run(False, 100)
    (graph, graph_greedy), engine = run(True, 100)
    assert any(k[2] == 128 for k in engine.decoder._slots)  # recorded with a buffer of 128 recent tokens
    assert graph == eager and graph_greedy == eager_greedy
    (short, _), _ = run(True, 64)
    assert short != graph


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_any_length_run_from_recordings_per_bucket(folders, dtype):
    """A prompt step - alone or beside decoding requests, ending its prompt or not - is
    replayed from a recording made for the bucket of its length: the rows between the
    portion's end and the bucket's belong to no request.  Prompts of many lengths, fed
    whole or in portions, give the tokens of an engine that records nothing, and the
    number of recordings stays small."""
    import infernum_b200 as ib
    model = ib.load_model(folders["B"], dtype=dtype)
    base = dict(max_batch_size=4, block_size=8, num_blocks=160, max_prefill_tokens=48, max_tokens_per_step=64)
    eager = ib.Engine(model, ib.BatchConfig(cuda_graphs=False, **base))
    graphs = ib.Engine(model, ib.BatchConfig(**base))
    plain = Plain(folders["B"])
    lengths = [16, 17, 31, 32, 33, 47, 48, 49, 95, 96, 97, 130, 20, 40, 45]
    prompts = [random_tokens(n, 320, 900 + n) for n in lengths]
    sampled = ib.SamplingParams(temperature=0.8, top_p=0.9, seed=2)
    opts = [ib.GenerateOptions(max_new_tokens=6, sampling=sampled if i % 4 == 1 else None) for i in range(len(prompts))]
    # one by one (every step is a prompt alone), then all together (portions beside decoded tokens)
    want = [eager.generate(p, o) for p, o in zip(prompts, opts)]
    for p, o, w in zip(prompts, opts, want):
        assert_same_up_to_ties(plain, p, graphs.generate(p, o), w, dtype, sampling=o.sampling)
    together = graphs.generate_batch(prompts, opts)
    for p, o, t, w in zip(prompts, opts, together, want):
        assert_same_up_to_ties(plain, p, t, w, dtype, sampling=o.sampling)
    keys = [k for k in graphs.decoder._slots if k[4] > 0]
    # (buckets of 16 for portions that end their prompts; a portion cut by the step's budget keeps its rows)
    assert keys and all(k[4] % 8 == 0 and k[4] <= 64 for k in keys) and len(keys) <= 32
    assert sum(1 for k in keys if graphs.decoder._slots[k].graph is not None) >= 4
    assert graphs.cache.free_pages() == [160] and graphs.cache.num_free_slots == 4
    graphs.runner.check_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_with_portions_are_launched_behind_the_step_in_flight(folders, dtype):
    """Many requests of all lengths through a small token budget: most steps hold
    decoded tokens beside one or two prompt portions (the end of one prompt and
    the start of the next).  Such a step is scheduled while the step before it
    runs, as if that step's tokens were known, and launched behind it with those
    tokens fed on the device.  A request that ends on a stop token leaves a row
    computed in vain, one that is cancelled too.  Everybody gets the tokens of
    an engine that records nothing and launches nothing ahead."""
    import infernum_b200 as ib
    model = ib.load_model(folders["B"], dtype=dtype)
    base = dict(max_batch_size=6, block_size=8, num_blocks=200, max_prefill_tokens=40, max_tokens_per_step=56)
    lengths = [70, 23, 5, 130, 41, 17, 64, 9, 88, 33, 2, 57]
    prompts = [random_tokens(n, 320, 500 + n) for n in lengths]
    sampled = ib.SamplingParams(temperature=0.8, top_p=0.9, seed=5)
    plainly = ib.Engine(model, ib.BatchConfig(cuda_graphs=False, **base))
    probe = plainly.generate(prompts[1], ib.GenerateOptions(max_new_tokens=20))

    def options():
        return [ib.GenerateOptions(max_new_tokens=14 + (i % 5), sampling=sampled if i % 3 == 1 else None,
                                   eos_token_id=probe[7] if i == 1 else None) for i in range(len(prompts))]

    def run(engine):
        handles = [engine.submit(p, o) for p, o in zip(prompts[:8], options()[:8])]
        for _ in range(6):
            engine.step()
        handles += [engine.submit(p, o) for p, o in zip(prompts[8:], options()[8:])]  # arrive later
        while len(handles[3].tokens) < 5:
            engine.step()
        engine.cancel(handles[3])
        engine.run_until_done(handles)
        while engine.has_work():
            engine.step()
        assert engine.cache.free_pages() == [200] and engine.cache.num_free_slots == 6
        return handles

    want = run(plainly)
    engine = ib.Engine(model, ib.BatchConfig(**base))
    seen = []
    launch = engine.decoder.launch

    def spy(slot, caches, tokens, sample=None, portions=None, feed_from=None, feed_rows=None, **more):
        seen.append((len(caches), len(portions or ()), feed_from is not None,
                     sum(1 for r in (feed_rows or ()) if r >= 0)))
        return launch(slot, caches, tokens, sample, portions=portions, feed_from=feed_from, feed_rows=feed_rows,
                      **more)

    engine.decoder.launch = spy
    got = run(engine)
    assert not engine.decoder._reads  # every launched step was read
    ahead = [s for s in seen if s[2]]
    # steps launched behind another: with one portion, with two, and with tokens fed on the device
    assert len(ahead) > 20 and any(s[1] == 1 and s[3] > 0 for s in ahead) and any(s[1] >= 2 for s in ahead)
    assert engine.stats.ahead_launched == len(ahead)
    assert engine.decoder.counts["replayed"] > 10
    plain = Plain(folders["B"])
    for k, (p, g, w) in enumerate(zip(prompts, got, want)):
        assert g.finish_reason == w.finish_reason
        n = min(len(g.tokens), len(w.tokens)) if k == 3 else max(len(g.tokens), len(w.tokens))
        assert_same_up_to_ties(plain, p, g.tokens[:n], w.tokens[:n], dtype, sampling=g.seq.options.sampling)
        if dtype == "float32" and k != 3:
            assert g.tokens == w.tokens
    engine.runner.check_errors()


# INFERNUM_TEST_MORE_SEEDS=N adds N seeds (from 100 on) whose batch settings are drawn from the seed
MORE_SEEDS = list(range(100, 100 + int(os.environ.get("INFERNUM_TEST_MORE_SEEDS", "0"))))


@pytest.mark.parametrize("seed", [1, 2, 3] + MORE_SEEDS)
def test_random_traffic_through_the_pipeline_equals_runs_alone(folders, seed):
    """Requests of random lengths and limits arrive at random moments; some stop
    on an end-of-sequence token, some are sampled (with and without a repetition
    penalty), some are cancelled, and the pages are so few that requests are
    preempted - while steps are scheduled and launched ahead of the tokens in
    flight.  In 32-bit every request gets, token for token, what it gets alone
    from an engine that records nothing and launches nothing ahead; no page or
    slot is lost.  Seeds 1 to 3 have fixed batch settings, under which requests
    must be preempted and steps launched ahead; further seeds draw the batch
    size, the pool, the portion and the token budget from the seed."""
    import random
    import infernum_b200 as ib
    rng = random.Random(seed)
    model = ib.load_model(folders["B"], dtype="float32")
    batch, pool, portion, budget = 5, 44, 24, 40
    if seed >= 100:
        draw = random.Random(seed * 7 + 1)
        batch, pool = draw.randint(2, 6), draw.randint(27, 60)
        portion, budget = draw.randint(4, 48), draw.randint(8, 64)
    base = dict(max_batch_size=batch, block_size=8, max_prefill_tokens=portion, max_tokens_per_step=budget,
                max_model_len=200)
    solo = ib.Engine(model, ib.BatchConfig(num_blocks=64, cuda_graphs=False, launch_ahead=False, **base))
    engine = ib.Engine(model, ib.BatchConfig(num_blocks=pool, **base))
    todo = []
    for i in range(26):
        prompt = random_tokens(rng.randint(1, 110), 320, 1000 * seed + i)
        kind = rng.random()
        sampling = None
        if kind < 0.25:
            sampling = ib.SamplingParams(temperature=0.9, top_p=0.9, seed=i)
        elif kind < 0.4:
            sampling = ib.SamplingParams(temperature=0.8, top_p=0.95, seed=i, repetition_penalty=1.2,
                                         repetition_penalty_window=16)
        n_new = rng.randint(1, 22)
        want = solo.generate(prompt, ib.GenerateOptions(max_new_tokens=n_new, sampling=sampling))
        eos = want[len(want) // 2] if len(want) > 3 and rng.random() < 0.3 else None
        if eos is not None:
            want = want[: want.index(eos)]
        todo.append((prompt, ib.GenerateOptions(max_new_tokens=n_new, sampling=sampling, eos_token_id=eos), want))
    live, done, cancelled = [], [], 0
    steps = 0
    while todo or engine.has_work():
        steps += 1
        assert steps < 3000
        if todo and rng.random() < 0.35:
            prompt, opts, want = todo.pop()
            live.append((engine.submit(prompt, opts), want))
        if live and rng.random() < 0.02:
            h, want = live[rng.randrange(len(live))]
            if not h.finished:
                engine.cancel(h)
                cancelled += 1
        engine.step()
    engine.run_until_done()
    for h, want in live:
        if h.finish_reason == ib.FinishReason.CANCELLED:
            assert h.tokens == want[: len(h.tokens)]
        else:
            assert h.tokens == want, (h.id, h.finish_reason)
    st = engine.stats
    if seed < 100:
        assert st.preemptions > 0 and st.ahead_launched > 30 and engine.decoder.counts["replayed"] > 30
    assert not engine.decoder._reads
    assert engine.cache.free_pages() == [pool] and engine.cache.num_free_slots == batch
    engine.runner.check_errors()


def test_cache_pools_sized_from_the_free_memory(folders, monkeypatch):
    """``num_blocks=None``: as many pages as the given share of the free memory
    holds; a request for pages that the device refuses says what a page costs
    (the refusal is played by a stand-in: no memory is taken)."""
    import infernum_b200 as ib
    from infernum_b200.errors import CacheError
    model = ib.load_model(folders["B"], dtype="bfloat16")
    free = torch.cuda.mem_get_info()[0]
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=2, block_size=16, num_blocks=None,
                                             cache_memory_fraction=0.01))
    per_page = engine.cache.bytes_per_token() * 16
    pages = engine.cache.num_pages
    assert pages > 100 and 0.008 * free < (pages + 1) * per_page <= 0.0101 * free
    prompt = random_tokens(9, 320, 5)
    assert engine.generate(prompt, ib.GenerateOptions(max_new_tokens=8)) == \
        ib.Engine(model, ib.BatchConfig(max_batch_size=2, block_size=16, num_blocks=8)).generate(
            prompt, ib.GenerateOptions(max_new_tokens=8))
    del engine
    torch.cuda.empty_cache()
    zeros = torch.zeros

    def refuse(shape, *args, **kwargs):
        if len(shape) == 4 and shape[0] > 1000:
            raise torch.cuda.OutOfMemoryError("stand-in")
        return zeros(shape, *args, **kwargs)

    monkeypatch.setattr(torch, "zeros", refuse)
    with pytest.raises(CacheError, match="do not fit the device"):
        ib.Engine(model, ib.BatchConfig(max_batch_size=2, block_size=16, num_blocks=5000))


def test_profile_mode_times_every_operation(folders, monkeypatch):
    """With profiling on (the switch ``INFERNUM_PROFILE=1`` sets at start-up) every
    operation's device time is summed per operation; the engine replays no
    recordings then, and generates what it generates otherwise."""
    import infernum_b200 as ib
    from infernum_b200.ops import core
    model = ib.load_model(folders["B"], dtype="bfloat16")
    cfg = ib.BatchConfig(max_batch_size=2, block_size=8, num_blocks=32)
    prompt = random_tokens(21, 320, 3)
    want = ib.Engine(model, cfg).generate(prompt, ib.GenerateOptions(max_new_tokens=6))
    monkeypatch.setattr(core, "PROFILE", True)
    core._profile_marks.clear()
    core._profile_totals.clear()
    engine = ib.Engine(model, cfg)
    assert engine.decoder is None
    assert engine.generate(prompt, ib.GenerateOptions(max_new_tokens=6)) == want
    totals = core.profile_collect()
    layers = len(model.layers)
    assert totals["add_rmsnorm"][0] == 6 * (2 * layers + 1) and totals["rope_append"][0] == 6 * layers
    assert all(calls > 0 and us >= 0 for calls, us in totals.values()) and totals["add_rmsnorm"][1] > 0
    assert any(k.startswith("attention") for k in totals) and any(k.startswith("gemm") for k in totals)
    text = core.profile_report()
    assert "share" in text and "add_rmsnorm" in text
    core._profile_totals.clear()
