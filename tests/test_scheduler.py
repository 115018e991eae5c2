"""The scheduler's decisions with a fake step (no GPU): admission order, the
token budget, portions, finishing, and what happens when pages run out."""
import os
from types import SimpleNamespace

import pytest

from infernum_b200.cache import CacheManager
from infernum_b200.engine.scheduler import BatchConfig, FinishReason, Phase, Scheduler
from infernum_b200.errors import SchedulingError
from infernum_b200.parts.base import PagedCacheSpec
from infernum_b200.sampling import GenerateOptions


def make(num_blocks=64, block_size=4, max_batch=4, chunk=8, budget=16, max_len=256):
    cfg = BatchConfig(max_batch_size=max_batch, max_prefill_tokens=chunk, block_size=block_size,
                      num_blocks=num_blocks, max_tokens_per_step=budget)
    need = SimpleNamespace(position=0, paged=PagedCacheSpec(1, 8, 0), state=None, cache_of=None)
    cache = CacheManager([need], page_size=block_size, num_pages=num_blocks, max_requests=max_batch)
    return Scheduler(cfg, cache, max_len), cache


def fake_token(seq):
    return (sum(seq.tokens) * 31 + len(seq.tokens)) % 97 + 3


def run_step(sched, cache, log=None):
    plan = sched.schedule()
    cache.check_invariants()
    for p in plan.portions:
        assert p.tokens == p.seq.tokens[p.seq.num_computed: p.seq.num_computed + p.count]
    sched.commit(plan, commit_cache=True)
    for p in plan.portions:
        if p.wants_logits:
            sched.append_token(p.seq, fake_token(p.seq))
    if log is not None:
        log.append(plan)
    return plan


def drain(sched, cache, limit=10000):
    log = []
    while sched.has_work():
        run_step(sched, cache, log)
        assert len(log) < limit, "the scheduler does not terminate"
    sched.schedule()  # reap
    cache.check_invariants()
    return log


def solo_tokens(prompt, n_new):
    sched, cache = make(num_blocks=max(256, (len(prompt) + n_new) // 4 + 2), max_len=max(256, len(prompt) + n_new))
    s = sched.add_request(prompt, GenerateOptions(max_new_tokens=n_new))
    drain(sched, cache)
    return s.generated_ids


def test_first_come_first_served_and_batch_limit():
    sched, cache = make(max_batch=2, budget=64, chunk=64)
    seqs = [sched.add_request([1] * 5, GenerateOptions(max_new_tokens=3)) for _ in range(4)]
    plan = run_step(sched, cache)
    assert [p.seq.id for p in plan.portions] == [0, 1]
    assert [s.phase for s in seqs] == [Phase.DECODE, Phase.DECODE, Phase.WAITING, Phase.WAITING]
    log = drain(sched, cache)
    assert all(s.finish_reason == FinishReason.LENGTH and len(s.generated_ids) == 3 for s in seqs)
    first_seen = []
    for plan in log:
        for p in plan.portions:
            if p.seq.id not in first_seen:
                first_seen.append(p.seq.id)
    assert first_seen == [0, 1, 2, 3] or first_seen == [2, 3]  # 0 and 1 started before the log


def test_budget_decodes_first_then_portions():
    sched, cache = make(budget=10, chunk=8, max_batch=4)
    a = sched.add_request([2] * 3, GenerateOptions(max_new_tokens=50))
    run_step(sched, cache)  # a prefilled, now decoding
    b = sched.add_request(list(range(3, 33)), GenerateOptions(max_new_tokens=2))
    plan = run_step(sched, cache)
    assert [(p.seq.id, p.count, p.wants_logits) for p in plan.portions] == [(0, 1, True), (1, 8, False)]
    plan = run_step(sched, cache)
    assert [(p.seq.id, p.start, p.count) for p in plan.portions] == [(0, 4, 1), (1, 8, 8)]
    c = sched.add_request([5] * 4, GenerateOptions(max_new_tokens=2))
    plan = run_step(sched, cache)  # 1 decode + 8 of b + 1 left for c
    assert [(p.seq.id, p.count) for p in plan.portions] == [(0, 1), (1, 8), (2, 1)]
    assert plan.num_tokens == 10
    plan = run_step(sched, cache)
    # b's last 6 tokens finish its prompt: it wants logits; c continues
    assert [(p.seq.id, p.count, p.wants_logits) for p in plan.portions] == \
        [(0, 1, True), (1, 6, True), (2, 3, True)]
    assert b.phase == Phase.DECODE and len(b.generated_ids) == 1
    drain(sched, cache)


def test_portions_cover_a_prompt_exactly_once():
    sched, cache = make(budget=7, chunk=5)
    prompt = list(range(10, 33))
    s = sched.add_request(prompt, GenerateOptions(max_new_tokens=1))
    log = drain(sched, cache)
    fed = [t for plan in log for p in plan.portions for t in p.tokens]
    assert fed == prompt
    assert [p.count for plan in log for p in plan.portions] == [5, 5, 5, 5, 3]
    assert s.finish_reason == FinishReason.LENGTH


def test_eos_is_neither_stored_nor_emitted():
    sched, cache = make()
    s = sched.add_request([1, 2, 3], GenerateOptions(max_new_tokens=10, eos_token_id=50))
    run_step(sched, cache)
    assert sched.append_token(s, 7) == 7
    assert sched.append_token(s, 50) is None
    assert s.finish_reason == FinishReason.STOP and s.generated_ids[-1] == 7
    t = sched.add_request([1], GenerateOptions(max_new_tokens=2, eos_token_id=50, ignore_eos=True))
    assert sched.append_token(t, 50) == 50 and not t.finished
    assert sched.append_token(t, 50) == 50 and t.finish_reason == FinishReason.LENGTH


def test_requests_that_can_never_run_are_refused():
    sched, _ = make(num_blocks=4, block_size=4, max_len=64)
    with pytest.raises(SchedulingError, match="pages"):
        sched.add_request([1] * 10, GenerateOptions(max_new_tokens=8))
    with pytest.raises(SchedulingError, match="longest"):
        sched.add_request([1] * 60, GenerateOptions(max_new_tokens=8))
    with pytest.raises(SchedulingError):
        sched.add_request([], GenerateOptions())
    sched.add_request([1] * 10, GenerateOptions(max_new_tokens=7))  # 16 cached at most: fits


def test_admission_waits_for_pages_without_skipping():
    sched, cache = make(num_blocks=6, block_size=4, budget=64, chunk=64)
    a = sched.add_request([1] * 16, GenerateOptions(max_new_tokens=2))
    big = sched.add_request([2] * 12, GenerateOptions(max_new_tokens=2))
    small = sched.add_request([3] * 2, GenerateOptions(max_new_tokens=2))
    plan = run_step(sched, cache)
    # a takes 4 pages; big's 3 pages do not fit in 2; small is not let past big
    assert [p.seq.id for p in plan.portions] == [a.id]
    assert big.phase == Phase.WAITING and small.phase == Phase.WAITING
    drain(sched, cache)
    assert all(s.finish_reason == FinishReason.LENGTH for s in (a, big, small))


def test_pages_run_out_the_youngest_is_preempted_and_output_is_unchanged():
    prompts = [[i + 1] * 9 for i in range(3)]
    want = [solo_tokens(p, 14) for p in prompts]
    # 3 requests x (9 + 13) tokens = 18 pages of 4 wanted, the pool has 12
    sched, cache = make(num_blocks=12, block_size=4, budget=64, chunk=64, max_batch=3)
    seqs = [sched.add_request(p, GenerateOptions(max_new_tokens=14)) for p in prompts]
    log = drain(sched, cache)
    assert sched.num_preemptions > 0
    victims = [v.id for plan in log for v in plan.preempted]
    assert victims and victims[0] == 2  # the most recently admitted goes first
    assert seqs[0].preemptions == 0  # the oldest is never a victim here
    assert [s.generated_ids for s in seqs] == want
    assert cache.free_pages() == [12] and cache.num_free_slots == 3
    assert cache.groups[0].pool.reuses > 0
    # a preempted request is recomputed from its tokens so far, in portions
    recompute = [p for plan in log for p in plan.portions if p.seq.id == 2 and p.start == 0]
    assert len(recompute) >= 2


def test_preempted_request_returns_to_the_front():
    sched, cache = make(num_blocks=6, block_size=4, budget=64, chunk=64, max_batch=2)
    a = sched.add_request([1] * 8, GenerateOptions(max_new_tokens=12))
    b = sched.add_request([2] * 8, GenerateOptions(max_new_tokens=12))
    c = sched.add_request([3] * 4, GenerateOptions(max_new_tokens=2))
    log = []
    while not b.preemptions:
        run_step(sched, cache, log)
    assert sched.waiting[0] is b and sched.waiting[1] is c
    assert b.cache is None and b.num_computed == 0 and b.phase == Phase.WAITING
    drain(sched, cache)
    assert len(a.generated_ids) == 12 and len(b.generated_ids) == 12 and len(c.generated_ids) == 2


def test_cancel_frees_pages():
    sched, cache = make()
    a = sched.add_request([1] * 9, GenerateOptions(max_new_tokens=20))
    b = sched.add_request([2] * 30, GenerateOptions(max_new_tokens=20))
    run_step(sched, cache)
    sched.cancel(b)  # mid-prefill
    run_step(sched, cache)
    assert b.cache is None and b.finish_reason == FinishReason.CANCELLED
    sched.cancel(a)  # mid-decode
    drain(sched, cache)
    assert cache.free_pages() == [64] and cache.num_free_slots == 4
    w = sched.add_request([3] * 3, GenerateOptions(max_new_tokens=2))
    sched.cancel(w)  # while waiting
    assert not sched.has_work() or drain(sched, cache) is not None
    assert w.finish_reason == FinishReason.CANCELLED and w.generated_ids == []


def test_many_requests_random_lengths_all_finish():
    import random
    rng = random.Random(5)
    sched, cache = make(num_blocks=40, block_size=4, budget=24, chunk=10, max_batch=4)
    reqs = []
    for i in range(25):
        p = [rng.randrange(3, 90) for _ in range(rng.randint(1, 40))]
        reqs.append((p, rng.randint(1, 30)))
    seqs = [sched.add_request(p, GenerateOptions(max_new_tokens=n)) for p, n in reqs]
    log = drain(sched, cache)
    for plan in log:
        assert plan.num_tokens <= 24
        assert len({p.seq.id for p in plan.portions}) == len(plan.portions)
    for s, (p, n) in zip(seqs, reqs):
        assert s.generated_ids == solo_tokens(p, n)
    assert cache.free_pages() == [40]


def test_a_preempted_request_waits_until_its_whole_recomputation_fits():
    sched, cache = make(num_blocks=16, block_size=4, budget=64, chunk=4, max_batch=2)
    a = sched.add_request([1] * 12, GenerateOptions(max_new_tokens=40))
    b = sched.add_request([2] * 12, GenerateOptions(max_new_tokens=40))
    log = []
    while not b.preemptions:
        run_step(sched, cache, log)
    # b now has its prompt and what it generated to recompute; a keeps growing.  While
    # fewer pages are free than b's tokens need, b stays in the queue even though a
    # first portion of 4 tokens would fit.
    readmitted_at = None
    for _ in range(200):
        sched._reap()  # what the round itself does first: finished requests give their pages back
        free_before = cache.free_pages()[0]
        need = cache.pages_for(b.num_tokens)
        plan = run_step(sched, cache, log)
        if b in plan.admitted:
            readmitted_at = (free_before, need)
            break
        if not sched.has_work():
            break
    assert readmitted_at is not None and readmitted_at[0] >= readmitted_at[1]
    drain(sched, cache)
    assert len(a.generated_ids) == 40 and len(b.generated_ids) == 40
    assert b.preemptions <= 2


def test_steps_a_little_above_a_multiple_of_the_tile_are_cut_back():
    """520 rows (a portion of 512 beside 8 decoded tokens) become 512; the 8 rows
    cut come with the next step, and every prompt is still covered exactly once."""
    cfg = BatchConfig(max_batch_size=16, max_prefill_tokens=512, block_size=16, num_blocks=1024,
                      max_tokens_per_step=2048, token_multiple=256)
    need = SimpleNamespace(position=0, paged=PagedCacheSpec(1, 8, 0), state=None, cache_of=None)
    cache = CacheManager([need], page_size=16, num_pages=1024, max_requests=16)
    sched = Scheduler(cfg, cache, 4096)
    opts = GenerateOptions(max_new_tokens=40, ignore_eos=True)
    short = [sched.add_request([5 + i] * 3, opts) for i in range(8)]
    run_step(sched, cache)  # the eight short prompts: 24 rows, left alone
    assert all(s.phase == Phase.DECODE for s in short)
    long = sched.add_request(list(range(3, 1403)), opts)
    plan = run_step(sched, cache)
    assert plan.num_tokens == 512  # 8 decoded tokens + 504 of the prompt, not 520
    assert sum(p.count for p in plan.portions if p.seq is long) == 504
    plan = run_step(sched, cache)
    assert plan.num_tokens == 512 and long.num_computed == 1008
    plan = run_step(sched, cache)  # 392 left + 8 = 400: far from a multiple, left alone
    assert plan.num_tokens == 400 and long.phase == Phase.DECODE
    drain(sched, cache)
    assert long.generated_ids == solo_tokens(list(range(3, 1403)), 40)
    cache.check_invariants()


def test_a_cut_portion_that_would_have_ended_its_prompt_asks_for_no_logits():
    cfg = BatchConfig(max_batch_size=4, max_prefill_tokens=600, block_size=16, num_blocks=256,
                      max_tokens_per_step=2048, token_multiple=256)
    need = SimpleNamespace(position=0, paged=PagedCacheSpec(1, 8, 0), state=None, cache_of=None)
    cache = CacheManager([need], page_size=16, num_pages=256, max_requests=4)
    sched = Scheduler(cfg, cache, 4096)
    seq = sched.add_request(list(range(3, 523)), GenerateOptions(max_new_tokens=2, ignore_eos=True))  # 520 tokens
    plan = run_step(sched, cache)
    assert plan.num_tokens == 512 and not plan.portions[0].wants_logits and not seq.generated_ids
    plan = run_step(sched, cache)
    assert plan.num_tokens == 8 and plan.portions[0].wants_logits and len(seq.generated_ids) == 1
    off = Scheduler(BatchConfig(max_batch_size=4, max_prefill_tokens=600, block_size=16, num_blocks=256,
                                token_multiple=0),
                    CacheManager([need], page_size=16, num_pages=256, max_requests=4), 4096)
    off.add_request(list(range(3, 523)), GenerateOptions(max_new_tokens=2, ignore_eos=True))
    assert off.schedule().num_tokens == 520


def test_the_next_step_can_be_planned_before_its_tokens_are_known():
    sched, cache = make(num_blocks=64, block_size=4, max_batch=4, chunk=8, budget=16)
    opts = GenerateOptions(max_new_tokens=6, ignore_eos=True)
    a = sched.add_request([5, 6, 7], opts)
    b = sched.add_request([8, 9], opts)
    run_step(sched, cache)  # prompts; both decode from here on
    # a decode step in flight: scheduled and committed, its tokens not yet appended
    plan = sched.schedule()
    sched.commit(plan, commit_cache=True)
    ahead = sched.plan_ahead(plan)
    assert ahead is not None and [p.seq for p in ahead.portions] == [a, b]
    assert [(p.start, p.count, p.wants_logits) for p in ahead.portions] == \
        [(a.num_computed, 1, True), (b.num_computed, 1, True)]
    assert a.pending == 1 and a.num_tokens == a.num_known + 1
    assert not sched.plan_still_holds(ahead)  # it feeds tokens nobody has seen yet
    for p in plan.portions:
        sched.append_token(p.seq, fake_token(p.seq))
    assert a.pending == 0 and sched.plan_still_holds(ahead)
    assert [p.tokens for p in ahead.portions] == [[a.generated_ids[-1]], [b.generated_ids[-1]]]
    cache.check_invariants()
    # a request that arrives joins a later step; one that ends voids the plan
    sched.add_request([1, 2, 3], opts)
    assert sched.plan_still_holds(ahead)
    sched.cancel(b)
    assert not sched.plan_still_holds(ahead)
    drain(sched, cache)
    assert a.generated_ids == solo_tokens([5, 6, 7], 6)


def test_planning_ahead_admits_portions_and_knows_the_limits():
    """The step planned ahead is a whole scheduling round: a prompt that ends in
    the step in flight decodes in the next, the next portion of a long prompt
    and a waiting request ride along.  A request whose token in flight is its
    last is known to end, so nothing is planned until that token is read."""
    sched, cache = make(num_blocks=64, block_size=4, max_batch=3, chunk=8, budget=16)
    opts = GenerateOptions(max_new_tokens=5, ignore_eos=True)
    a = sched.add_request([5, 6, 7], opts)
    b = sched.add_request(list(range(3, 23)), opts)       # 20 tokens: portions of 8, 8, 4
    plan = sched.schedule()                                 # a whole, b's first portion
    sched.commit(plan, commit_cache=True)
    c = sched.add_request([9, 9], opts)
    ahead = sched.plan_ahead(plan)
    assert [(p.seq, p.start, p.count, p.wants_logits) for p in ahead.portions] == \
        [(a, 3, 1, True), (b, 8, 8, False), (c, 0, 2, True)]
    assert a.phase == Phase.DECODE and a.pending == 1 and b.pending == 0
    cache.check_invariants()
    for p in plan.portions:
        if p.wants_logits:
            sched.append_token(p.seq, fake_token(p.seq))
    assert sched.plan_still_holds(ahead)
    drain(sched, cache)
    assert a.generated_ids == solo_tokens([5, 6, 7], 5) and len(b.generated_ids) == 5
    # the limit: a request whose token in flight is its last has no row in the step planned ahead;
    # alone, nothing is planned; its slot is free for the next request only when the token has come
    sched, cache = make(num_blocks=64, block_size=4, max_batch=2)
    a = sched.add_request([5, 6, 7], GenerateOptions(max_new_tokens=2, ignore_eos=True))
    run_step(sched, cache)
    plan = sched.schedule()
    sched.commit(plan, commit_cache=True)
    assert sched.plan_ahead(plan) is None and not a.finished
    b = sched.add_request([8, 9, 10, 11], GenerateOptions(max_new_tokens=3, ignore_eos=True))
    c = sched.add_request([1, 2], GenerateOptions(max_new_tokens=3, ignore_eos=True))
    ahead = sched.plan_ahead(plan)
    assert [p.seq for p in ahead.portions] == [b] and a.ends_in_flight and c.phase == Phase.WAITING
    for p in plan.portions:
        sched.append_token(p.seq, fake_token(p.seq))
    assert a.finished and a.finish_reason == FinishReason.LENGTH and sched.plan_still_holds(ahead)
    drain(sched, cache)
    assert b.generated_ids == solo_tokens([8, 9, 10, 11], 3) and c.generated_ids == solo_tokens([1, 2], 3)
    # one slot only: the request that waits cannot come in before the token in flight has
    # arrived, and the one that is about to end is neither preempted nor failed for it
    sched, cache = make(num_blocks=64, block_size=4, max_batch=1)
    a = sched.add_request([5, 6, 7], GenerateOptions(max_new_tokens=2, ignore_eos=True))
    b = sched.add_request([8, 9], GenerateOptions(max_new_tokens=2, ignore_eos=True))
    run_step(sched, cache)
    plan = sched.schedule()
    sched.commit(plan, commit_cache=True)
    assert sched.plan_ahead(plan) is None and not a.finished and a.cache is not None
    for p in plan.portions:
        sched.append_token(p.seq, fake_token(p.seq))
    drain(sched, cache)
    assert a.finish_reason == b.finish_reason == FinishReason.LENGTH and b.generated_ids == solo_tokens([8, 9], 2)


def test_planning_ahead_takes_pages_like_any_round():
    """Two requests fill the pool; the round planned ahead needs a page more, so
    the younger request is preempted while its token is still in flight.  The
    token is kept when it arrives, the request waits (it is not let back in
    before that), is computed again and ends with the tokens it gets alone."""
    sched, cache = make(num_blocks=4, block_size=4)
    opts = GenerateOptions(max_new_tokens=8, ignore_eos=True)
    a = sched.add_request([1] * 7, opts)
    b = sched.add_request([2] * 7, opts)
    run_step(sched, cache)           # 7 tokens each: two pages each, the pool is full
    plan = sched.schedule()          # token 8 fits the pages held
    sched.commit(plan, commit_cache=True)
    ahead = sched.plan_ahead(plan)   # token 9 needs a fifth page
    assert [p.seq for p in ahead.portions] == [a] and ahead.preempted == [b]
    assert b.phase == Phase.WAITING and b.pending == 1 and b.cache is None
    cache.check_invariants()
    for p in plan.portions:
        sched.append_token(p.seq, fake_token(p.seq))
    assert b.phase == Phase.WAITING and b.pending == 0 and len(b.generated_ids) == 2
    assert sched.plan_still_holds(ahead)
    drain(sched, cache)
    assert a.generated_ids == solo_tokens([1] * 7, 8) and b.generated_ids == solo_tokens([2] * 7, 8)
    assert cache.free_pages() == [4]


# INFERNUM_TEST_MORE_SEEDS=N adds N seeds (from 100 on) with sizes drawn from the seed
MORE_SEEDS = list(range(100, 100 + int(os.environ.get("INFERNUM_TEST_MORE_SEEDS", "0"))))


@pytest.mark.parametrize("seed", [11] + MORE_SEEDS)
def test_planning_ahead_under_random_arrivals_ends_and_tight_pages(seed):
    """The engine's way of driving the scheduler - schedule the next step while
    one is in flight, as if its tokens were there; run it at once if it only
    needs them on the device, else when they have come and the plan still
    holds - under random prompt lengths, arrivals between steps,
    end-of-sequence tokens and so few pages that requests are preempted: every
    request gets the tokens it gets alone, no page is lost, and plans made
    ahead are launched, used later and voided.  Seed 11 has fixed sizes and must
    show all three fates of a plan; further seeds draw the page size, the batch,
    the portion, the budget, the length limit and the pool from the seed."""
    import random
    rng = random.Random(seed)
    if seed == 11:
        nb, bs, max_batch, chunk, budget, max_len = 48, 4, 5, 9, 20, 200
        todo = [([rng.randrange(3, 90) for _ in range(rng.randint(1, 40))], rng.randint(1, 25)) for _ in range(40)]
    else:
        bs = rng.choice([2, 4, 8])
        max_batch = rng.randint(1, 6)
        chunk = rng.randint(2, 24)
        budget = rng.randint(max(2, max_batch), 40)
        max_len = rng.choice([60, 120, 200])
        nb = rng.randint(max_len // bs + 2, 3 * max_len // bs)
        todo = [([rng.randrange(3, 90) for _ in range(rng.randint(1, min(60, max_len - 2)))], rng.randint(1, 30))
                for _ in range(rng.randint(5, 40))]
    sched, cache = make(num_blocks=nb, block_size=bs, max_batch=max_batch, chunk=chunk, budget=budget, max_len=max_len)
    expect, seqs = [], []
    launched = used = voided = 0
    ahead = None  # (plan, launched)
    steps = 0

    def land(plan):
        for p in plan.portions:
            if p.wants_logits:
                if p.seq.finished:
                    p.seq.pending = 0  # (computed in vain)
                else:
                    sched.append_token(p.seq, fake_token(p.seq))

    while todo or sched.has_work() or ahead is not None:
        steps += 1
        assert steps < 20000
        if todo and rng.random() < 0.3:
            p, n = todo.pop()
            want = solo_tokens(p, n)[: max(0, max_len - len(p))]  # the length limit ends a request too
            eos = want[len(want) // 2] if (len(want) > 3 and rng.random() < 0.4) else None
            try:
                seqs.append(sched.add_request(p, GenerateOptions(max_new_tokens=n, eos_token_id=eos)))
            except SchedulingError:
                continue  # it could never run here
            expect.append(want if eos is None else want[: want.index(eos)])
        plan, in_flight = None, False
        if ahead is not None:
            plan, in_flight = ahead
            ahead = None
            if in_flight:
                launched += 1
            elif sched.plan_still_holds(plan):
                used += 1
            else:
                plan, voided = None, voided + 1
        if plan is None:
            plan = sched.schedule()
        cache.check_invariants()
        if not in_flight:
            for p in plan.portions:  # run from the host: every token is known
                assert p.tokens == p.seq.tokens[p.seq.num_computed: p.seq.num_computed + p.count]
        if not plan.portions:
            continue
        sched.commit(plan, commit_cache=True)
        nxt = sched.plan_ahead(plan)
        cache.check_invariants()
        if nxt is not None:
            # launched at once when every portion's tokens are known (what the engine
            # runs from recordings; seed 11 keeps to one portion beside the decoded
            # tokens); else kept for later
            many = [p for p in nxt.portions if p.count > 1 or not p.wants_logits]
            now = ((len(many) <= 1 or seed != 11) and all(not p.seq.pending for p in many)
                   and rng.random() < 0.8)
            if now:
                for p in nxt.portions:  # a token in flight is fed on the device, the others are known
                    assert p.seq.pending == (1 if p.start + p.count > p.seq.num_known else 0)
            ahead = (nxt, now)
        land(plan)  # the tokens of `plan` arrive
    sched.schedule()
    cache.check_invariants()
    assert [s.generated_ids for s in seqs] == expect
    assert cache.free_pages() == [nb]
    if seed == 11:
        assert launched > 20 and used > 3 and voided > 0, (launched, used, voided)


def test_leftover_budget_is_not_spent_on_a_sliver_of_a_prompt():
    """Beside a full portion, what is left of the budget starts no portion of a
    few tokens (unless they finish the prompt); alone, or when they end their
    prompt, few tokens are taken as they come."""
    cfg = BatchConfig(max_batch_size=8, max_prefill_tokens=512, block_size=16, num_blocks=1024,
                      max_tokens_per_step=560, token_multiple=0, min_portion_tokens=64)
    need = SimpleNamespace(position=0, paged=PagedCacheSpec(1, 8, 0), state=None, cache_of=None)
    cache = CacheManager([need], page_size=16, num_pages=1024, max_requests=8)
    sched = Scheduler(cfg, cache, 4096)
    opts = GenerateOptions(max_new_tokens=4, ignore_eos=True)
    a = sched.add_request(list(range(3, 1203)), opts)   # 1200 tokens
    b = sched.add_request(list(range(3, 903)), opts)    # 900 tokens
    c = sched.add_request([7] * 30, opts)
    plan = run_step(sched, cache)
    # a takes 512; 48 are left: no sliver of b (it would not end b's prompt) ...
    assert [(p.seq.id, p.count) for p in plan.portions] == [(a.id, 512)]
    assert b.phase == Phase.WAITING and c.phase == Phase.WAITING  # ... and nobody is skipped
    run_step(sched, cache)
    plan = run_step(sched, cache)  # a's last 176 tokens; 384 left: a real portion of b
    assert [(p.seq.id, p.count) for p in plan.portions] == [(a.id, 176), (b.id, 384)]
    plan = run_step(sched, cache)  # a decodes, b takes 512; c's 30 tokens end its prompt: taken
    assert [(p.seq.id, p.count) for p in plan.portions] == [(a.id, 1), (b.id, 512), (c.id, 30)]
    drain(sched, cache)
    assert a.generated_ids == solo_tokens(list(range(3, 1203)), 4)
    cache.check_invariants()


def test_last_tokens_of_a_request():
    from infernum_b200.engine.scheduler import Sequence_
    s = Sequence_(0, [1, 2, 3, 4, 5], GenerateOptions())
    assert s.last_tokens(3) == [3, 4, 5] and s.last_tokens(9) == [1, 2, 3, 4, 5] and s.last_tokens(0) == []
    s.generated_ids = [7, 8]
    assert s.last_tokens(1) == [8] and s.last_tokens(2) == [7, 8] and s.last_tokens(4) == [4, 5, 7, 8]
    assert s.last_tokens(99) == s.tokens
