"""Continuous batching: admits requests, cuts prompts into portions under a
token budget, decodes, finishes, frees - and decides what happens when pages
run out.

What is kept from the reference's scheduler
(infernum-runtime/src/scheduler.rs:197-404): a FIFO ``waiting`` queue and a
``running`` list; phases Waiting -> Prefill -> Decode -> Finished(reason);
admission first come first served and never skipping the head of the queue;
``max_batch_size`` running requests at most; ``max_prefill_tokens`` caps one
request's portion; finished requests are removed and their pages freed at the
start of the next scheduling round (:289-305).

What is different: the reference emits only the first portion of a long prompt
and never the rest (:341-352, ``continue_prefill`` has no caller), allocates a
whole prompt's blocks at admission, and on exhaustion during decode silently
drops the new block (infernum-runtime/src/engine.rs:476-480).  Here

  * a request is a sequence of tokens (prompt, then what it generated) of which
    a prefix is *computed* (in the cache); every step feeds the next portion,
    and a decode step is simply a portion of one token;
  * each step has a budget ``max_tokens_per_step``: decoding requests first
    (one token each), then running prompts in admission order, then new
    admissions;
  * pages are taken per step for exactly the step's tokens;
  * when a decoding request needs a page and none is free, the most recently
    admitted running request is *preempted*: its pages and slot are given
    back, and it returns to the front of the waiting queue to be recomputed
    from its tokens so far.  Its output does not change: greedy selection is a
    function of the logits, and a sampled token's random number is a function
    of (seed, tokens generated so far).  A prompt portion that does not fit is
    shortened or waits; only if nothing at all can run is a victim preempted
    for it.  A request that can never fit is refused when it is added.
"""

from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence

from ..cache.manager import CacheManager, RequestCache
from ..errors import SchedulingError
from ..sampling.params import GenerateOptions


class FinishReason(enum.Enum):
    STOP = "stop"  # the end-of-sequence token was selected
    LENGTH = "length"  # max_new_tokens reached
    CANCELLED = "cancelled"
    ERROR = "error"


class Phase(enum.Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODE = "decode"
    FINISHED = "finished"


@dataclass
class BatchConfig:
    """Engine limits; the first four are the reference's ``BatchConfig`` with
    its defaults (infernum-runtime/src/scheduler.rs:73-95)."""

    max_batch_size: int = 32
    max_prefill_tokens: int = 512
    block_size: int = 16
    # pages of every cache group's pool, or a list with one number per group; None: as many as
    # `cache_memory_fraction` of the device's free memory holds
    num_blocks: Optional[int] = 1024
    cache_memory_fraction: float = 0.9
    max_tokens_per_step: int = 2048
    max_model_len: Optional[int] = None  # default: the model's max_position_embeddings
    cuda_graphs: bool = True  # replay a recorded graph while the same requests decode
    # The kernels for prompts work on tiles of so many rows.  A step with prompt
    # portions whose row count lies a little above a multiple of it (by at most
    # 1/16) is cut back to that multiple; the rows cut come with the next step.
    # 0: leave steps as they are.
    token_multiple: int = 256
    # Budget that is left over beside a prompt portion of this step is not spent on a
    # further portion of fewer tokens than this (and than an eighth of
    # max_prefill_tokens) unless it finishes its prompt: a sliver costs a whole pass
    # over the weights' tiles, and without it steps keep recurring shapes.
    min_portion_tokens: int = 64
    # Launch the next decode step behind the one in flight, before its tokens are
    # read, whenever that step is certain but for those tokens (nobody waits,
    # nobody reaches a length limit, pages are there).  A request that ends on a
    # token nobody could foresee (end-of-sequence, cancel) then has computed one
    # token in vain.
    launch_ahead: bool = True


@dataclass
class Sequence_:
    id: int
    prompt_ids: List[int]
    options: GenerateOptions
    generated_ids: List[int] = field(default_factory=list)
    phase: Phase = Phase.WAITING
    finish_reason: Optional[FinishReason] = None
    num_computed: int = 0  # tokens whose keys/values are in the cache
    cache: Optional[RequestCache] = None
    admitted_at: int = -1  # admission counter value, for "most recently admitted"
    preemptions: int = 0
    error: Optional[str] = None
    # 1 while the token a step in flight selects for this request is not known yet: the
    # request is scheduled as if it had it (its value is fed on the device)
    pending: int = 0

    @property
    def tokens(self) -> List[int]:
        """The tokens known so far (one in flight is not among them)."""
        return self.prompt_ids + self.generated_ids

    @property
    def num_known(self) -> int:
        return len(self.prompt_ids) + len(self.generated_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.generated_ids) + self.pending

    def last_tokens(self, n: int) -> List[int]:
        """The last ``n`` known tokens (fewer if there are fewer), without building the whole list."""
        if n <= 0:
            return []
        g = self.generated_ids
        if len(g) >= n:
            return g[len(g) - n:]
        need = n - len(g)
        return self.prompt_ids[max(0, len(self.prompt_ids) - need):] + g

    def token_at(self, i: int) -> int:
        n = len(self.prompt_ids)
        return self.prompt_ids[i] if i < n else self.generated_ids[i - n]

    def token_range(self, start: int, stop: int) -> List[int]:
        n = len(self.prompt_ids)
        if stop <= n:
            return self.prompt_ids[start:stop]
        if start >= n:
            return self.generated_ids[start - n: stop - n]
        return self.prompt_ids[start:] + self.generated_ids[: stop - n]

    @property
    def remaining(self) -> int:
        return self.num_tokens - self.num_computed

    @property
    def ends_in_flight(self) -> bool:
        """The token in flight is the last one this request may have: whatever it
        is, the request ends when it arrives, and takes no part in a step
        planned before that."""
        return bool(self.pending) and len(self.generated_ids) + self.pending >= self.options.max_new_tokens

    @property
    def finished(self) -> bool:
        return self.phase == Phase.FINISHED


@dataclass
class Portion:
    seq: Sequence_
    start: int  # index of the first token fed
    count: int
    wants_logits: bool  # the portion reaches the end of the request's tokens

    @property
    def tokens(self) -> List[int]:
        return self.seq.token_range(self.start, self.start + self.count)


@dataclass
class StepPlan:
    portions: List[Portion] = field(default_factory=list)
    preempted: List[Sequence_] = field(default_factory=list)
    admitted: List[Sequence_] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(p.count for p in self.portions)


class Scheduler:
    def __init__(self, config: BatchConfig, cache: CacheManager, max_model_len: int):
        self.config = config
        self.cache = cache
        self.max_model_len = int(max_model_len)
        self.waiting: Deque[Sequence_] = deque()
        self.running: List[Sequence_] = []
        self._next_id = 0
        self._admissions = 0
        self.num_preemptions = 0

    # ---- requests --------------------------------------------------------------
    def add_request(self, prompt_ids: Sequence[int], options: GenerateOptions) -> Sequence_:
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise SchedulingError("a request needs at least one prompt token")
        if options.max_new_tokens < 1:
            raise SchedulingError("max_new_tokens must be at least 1")
        total = len(prompt) + options.max_new_tokens
        if total > self.max_model_len:
            raise SchedulingError(
                f"prompt ({len(prompt)}) + max_new_tokens ({options.max_new_tokens}) exceeds the "
                f"longest sequence the engine takes ({self.max_model_len})")
        # the last generated token is never fed, so total - 1 tokens are cached at most
        if not self.cache.could_ever_hold(total - 1, self.config.max_prefill_tokens):
            raise SchedulingError(
                f"the request needs {self.cache.peak_pages(total - 1, self.config.max_prefill_tokens)} pages "
                f"(per cache group), the pools have {self.cache.group_pages}: it could never run")
        seq = Sequence_(self._next_id, prompt, options)
        self._next_id += 1
        self.waiting.append(seq)
        return seq

    def cancel(self, seq: Sequence_) -> None:
        if not seq.finished:
            self._finish(seq, FinishReason.CANCELLED)

    def has_work(self) -> bool:
        return bool(self.waiting) or any(not s.finished for s in self.running)

    # ---- one scheduling round --------------------------------------------------
    def schedule(self, ahead: bool = False) -> StepPlan:
        plan = StepPlan()
        self._reap()
        while True:
            self._fill(plan)
            if plan.portions or not self.running or ahead:
                # (a round planned ahead in which nothing fits is left to the round that
                # knows the tokens in flight: a request may be about to end and make room)
                break
            # Nothing fits although requests are running: make room.
            victim = self._most_recent(exclude=None)
            if len(self.running) == 1:
                # cannot happen for a request that passed add_request; guard anyway
                self._finish(victim, FinishReason.ERROR, "the page pool is too small for this request")
                self._reap()
                break
            self._preempt(victim, plan)
        self._trim_to_multiple(plan)
        return plan

    def plan_ahead(self, in_flight: StepPlan) -> Optional[StepPlan]:
        """The step after ``in_flight``, scheduled while that one still runs and
        before the tokens it selects are known.  What the scheduler decides
        depends on how many tokens a request has, not on which, with two
        exceptions: a request may end on the token in flight (end-of-sequence),
        and one that reaches its length limit with it ends for certain.  The
        second is known beforehand: such a request gets no row in the planned
        step (its pages go back when its token has arrived).  The first is not:
        a request that turns out to have ended has a row in the planned step
        that was computed in vain; its pages go back at the next round, as always.

        Every request that gets a token from ``in_flight`` is marked as having
        one token more (``pending``); the round then runs as ``schedule`` does,
        admissions and preemptions included.  The plan holds no token values:
        the caller feeds the tokens in flight on the device, or waits for them
        and checks the plan with ``plan_still_holds``.  Whatever was reserved or
        admitted for a plan that is not used stays with its requests."""
        coming = []
        for p in in_flight.portions:
            seq = p.seq
            if not p.wants_logits or seq.finished or seq.cache is None:
                continue
            if seq.num_computed + 1 >= self.max_model_len:
                return None
            coming.append(seq)
        if not self.waiting and not any(s.phase == Phase.PREFILL for s in self.running) and all(
                len(s.generated_ids) + 1 >= s.options.max_new_tokens for s in coming):
            return None  # nothing would be left to run
        for seq in coming:
            seq.pending = 1
            seq.phase = Phase.DECODE
        plan = self.schedule(ahead=True)
        return plan if plan.portions else None

    def plan_still_holds(self, plan: StepPlan) -> bool:
        """Whether a plan of ``plan_ahead`` that was not launched can run now that
        the tokens of the step before it are appended: nobody in it has ended or
        lost its pages, and every token it feeds is known."""
        return bool(plan.portions) and all(
            not p.seq.finished and p.seq.cache is not None and p.seq.pending == 0
            and p.start == p.seq.num_computed and p.start + p.count <= p.seq.num_known
            for p in plan.portions)

    def _trim_to_multiple(self, plan: StepPlan) -> None:
        m = self.config.token_multiple
        total = plan.num_tokens
        if m <= 0 or total <= m:
            return
        extra = total % m
        if extra == 0 or extra * 16 > total:
            return
        # the last prompt portion that stays a portion of at least two tokens
        for p in reversed(plan.portions):
            if p.count >= extra + 2:
                p.count -= extra           # its pages stay reserved for the next step
                p.wants_logits = False     # it no longer reaches the request's last token
                return

    def _fill(self, plan: StepPlan) -> None:
        cfg = self.config
        budget = cfg.max_tokens_per_step
        plan.portions.clear()
        scheduled = set()
        # 1. decoding requests, oldest first; preempt the youngest for pages
        for seq in sorted(self.running, key=lambda s: s.admitted_at):
            if seq.finished or seq.phase != Phase.DECODE or seq.cache is None or seq.ends_in_flight:
                continue
            if budget <= 0:
                break
            while not self.cache.can_extend(seq.cache, self._to_reserve(seq, 1)):
                victim = self._most_recent(exclude=scheduled)
                if victim is None:
                    break
                self._preempt(victim, plan)
                if victim is seq:
                    break
            if seq.cache is None or not self.cache.can_extend(seq.cache, self._to_reserve(seq, 1)):
                continue
            self.cache.extend(seq.cache, self._to_reserve(seq, 1))
            plan.portions.append(Portion(seq, seq.num_computed, 1, True))
            scheduled.add(seq.id)
            budget -= 1
        # 2. running prompts (and recomputations), oldest first
        for seq in sorted(self.running, key=lambda s: s.admitted_at):
            if seq.finished or seq.phase != Phase.PREFILL or seq.cache is None:
                continue
            budget -= self._schedule_portion(seq, budget, plan)
        # 3. admissions, first come first served, never skipping
        #    (none in a round that preempted: the victim would come straight back)
        while self.waiting and budget > 0 and len(self.running) < cfg.max_batch_size \
                and self.cache.num_free_slots > 0 and not plan.preempted:
            seq = self.waiting[0]
            if seq.finished:  # cancelled while waiting
                self.waiting.popleft()
                continue
            if seq.pending:  # preempted while its latest token is in flight: that token comes first
                break
            first = min(seq.remaining, cfg.max_prefill_tokens, budget)
            if self._sliver(first, seq, plan):
                break
            # A request that was preempted comes back only when all it has to
            # recompute fits: let back in for one portion it would run out of pages
            # again at once and be preempted again.
            need = seq.remaining if seq.preemptions else first
            fit = self._fit(None, need)
            if fit < need and (self.running or fit <= 0):
                break  # the head request does not fit yet: wait, skip nobody
            self.waiting.popleft()
            seq.cache = self.cache.admit(seq.id)
            seq.phase = Phase.PREFILL
            seq.num_computed = 0
            seq.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(seq)
            plan.admitted.append(seq)
            budget -= self._schedule_portion(seq, budget, plan)

    def _sliver(self, count: int, seq: Sequence_, plan: StepPlan) -> bool:
        """Whether ``count`` tokens of ``seq`` would be a sliver of a portion beside
        another prompt portion of this step (see ``BatchConfig.min_portion_tokens``)."""
        least = min(self.config.min_portion_tokens, self.config.max_prefill_tokens // 8)
        return count < seq.remaining and count < least and any(p.count > 1 for p in plan.portions)

    def _to_reserve(self, seq: Sequence_, count: int) -> int:
        """Tokens to add to the pages held so that ``count`` more can be computed."""
        return max(0, seq.num_computed + count - seq.cache.reserved_tokens)

    def _fit(self, rc: Optional[RequestCache], count: int) -> int:
        """How many of ``count`` new tokens fit the free pages right now."""
        ps = self.cache.page_size
        free = min(self.cache.free_pages()) if self.cache.groups else 1 << 30
        if rc is None:
            return min(count, free * ps)
        slack = max(len(t) for t in rc.tables) * ps - rc.reserved_tokens if rc.tables else 0
        return min(count, slack + free * ps)

    def _schedule_portion(self, seq: Sequence_, budget: int, plan: StepPlan) -> int:
        if budget <= 0 or seq.remaining <= 0:
            return 0
        count = min(seq.remaining, self.config.max_prefill_tokens, budget)
        count = self._fit(seq.cache, self._to_reserve(seq, count)) + \
            (count - self._to_reserve(seq, count))
        count = min(count, seq.remaining)
        if count <= 0 or self._sliver(count, seq, plan):
            return 0
        self.cache.extend(seq.cache, self._to_reserve(seq, count))
        plan.portions.append(Portion(seq, seq.num_computed, count,
                                     seq.num_computed + count == seq.num_tokens))
        return count

    # ---- after the step ran ------------------------------------------------------
    def commit(self, plan: StepPlan, commit_cache: bool = False) -> None:
        """The step ran: its tokens are cached.  The step function counts them
        in the cache manager itself; ``commit_cache`` does it here for callers
        that run no real step."""
        for p in plan.portions:
            seq = p.seq
            if seq.cache is None:
                continue
            if commit_cache:
                self.cache.commit(seq.cache, p.count)
            seq.num_computed += p.count

    def append_token(self, seq: Sequence_, token: int) -> Optional[int]:
        """Takes the token selected for ``seq``; returns it if it is emitted.
        End-of-sequence is neither stored nor emitted; the token selected
        after the prompt counts as the first generated one
        (infernum-runtime/src/engine.rs:445-481, 286-288)."""
        seq.pending = 0
        if seq.finished:
            return None
        opts = seq.options
        if opts.eos_token_id is not None and token == opts.eos_token_id and not opts.ignore_eos:
            self._finish(seq, FinishReason.STOP)
            return None
        seq.generated_ids.append(int(token))
        if seq.phase != Phase.WAITING:  # (preempted while this token was in flight: it waits on)
            seq.phase = Phase.DECODE
        if len(seq.generated_ids) >= opts.max_new_tokens:
            self._finish(seq, FinishReason.LENGTH)
        return int(token)

    # ---- internals ---------------------------------------------------------------
    def _most_recent(self, exclude) -> Optional[Sequence_]:
        cands = [s for s in self.running
                 if not s.finished and s.cache is not None and (not exclude or s.id not in exclude)]
        return max(cands, key=lambda s: s.admitted_at) if cands else None

    def _preempt(self, victim: Sequence_, plan: StepPlan) -> None:
        plan.portions[:] = [p for p in plan.portions if p.seq is not victim]
        self.cache.release(victim.cache)
        victim.cache = None
        victim.num_computed = 0
        victim.phase = Phase.WAITING
        victim.preemptions += 1
        self.num_preemptions += 1
        self.running.remove(victim)
        self.waiting.appendleft(victim)
        plan.preempted.append(victim)

    def _finish(self, seq: Sequence_, reason: FinishReason, error: Optional[str] = None) -> None:
        seq.phase = Phase.FINISHED
        seq.finish_reason = reason
        seq.error = error

    def _reap(self) -> None:
        """Removes finished requests and gives their pages and slots back."""
        keep = []
        for seq in self.running:
            if seq.finished:
                if seq.cache is not None:
                    self.cache.release(seq.cache)
                    seq.cache = None
            else:
                keep.append(seq)
        self.running = keep
        while self.waiting and self.waiting[0].finished:
            self.waiting.popleft()
