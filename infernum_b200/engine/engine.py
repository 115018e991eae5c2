"""The token engine: requests in, tokens out.

It plays the role of the reference's ``Engine``
(infernum-runtime/src/engine.rs:39-170: ``new``/``with_config``, ``submit``,
``generate``, ``generate_stream``) and of its worker loop (:177-238), but as a
loop the caller drives: ``step()`` runs one scheduling round and one model
step, ``generate*`` run until their requests are done.  Events have the
reference's kinds: a token, finished(reason), error
(infernum-runtime/src/scheduler.rs:37-44).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import CacheManager
from ..errors import InfernumError
from ..sampling.params import GenerateOptions
from ..sampling.sampler import Sampler, pack_choices, recent_window
from .decode import DecodeRunner, bucket_for
from .scheduler import BatchConfig, FinishReason, Scheduler, Sequence_, StepPlan
from .step import ModelRunner, StepEntry


@dataclass
class GenerationEvent:
    kind: str  # "token" | "finished" | "error"
    token: Optional[int] = None
    reason: Optional[FinishReason] = None
    message: Optional[str] = None


@dataclass
class RequestHandle:
    """A submitted request: its tokens so far and its events."""

    seq: Sequence_
    events: List[GenerationEvent] = field(default_factory=list)
    _reported_finish: bool = False

    @property
    def id(self) -> int:
        return self.seq.id

    @property
    def tokens(self) -> List[int]:
        return list(self.seq.generated_ids)

    @property
    def finished(self) -> bool:
        return self.seq.finished

    @property
    def finish_reason(self) -> Optional[FinishReason]:
        return self.seq.finish_reason


@dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    generated_tokens: int = 0
    step_seconds: float = 0.0
    wait_seconds: float = 0.0  # of those, spent waiting for the device's results (the rest is the host's own work)
    ahead_used: int = 0    # decode steps that ran from a plan made while the step before them ran
    ahead_voided: int = 0  # such plans dropped because a request ended or arrived meanwhile
    ahead_launched: int = 0  # of the former, those launched before the step before them was read


class Engine:
    def __init__(self, model, config: Optional[BatchConfig] = None):
        self.model = model
        self.config = config or BatchConfig()
        cfg = self.config
        rt = model.rt
        self.cache = CacheManager(model.cache_needs(), page_size=cfg.block_size,
                                  num_pages=cfg.num_blocks, max_requests=cfg.max_batch_size,
                                  dtype=rt.dtype, device=rt.device)
        self.runner = ModelRunner(model, self.cache, max_rows=cfg.max_tokens_per_step,
                                  max_entries=cfg.max_batch_size)
        max_len = cfg.max_model_len or model.spec.max_position
        self.scheduler = Scheduler(cfg, self.cache, max_len)
        self.sampler = Sampler(rt.device)
        self.stats = EngineStats()
        self._handles: Dict[int, RequestHandle] = {}
        self.decoder = DecodeRunner(self.runner, max_len, use_graph=True) if cfg.cuda_graphs and model.replayable else None
        # the next decode step, planned and prepared while the one before it ran
        # (plan, prepared buffers, whether it is on the GPU already)
        self._ahead: Optional[Tuple[StepPlan, object, bool]] = None
        self.h2d_bytes = 0  # bytes of step inputs copied to the device so far
        self.d2h_bytes = 0  # bytes of step results read back so far

    @classmethod
    def with_config(cls, model, config: BatchConfig) -> "Engine":
        return cls(model, config)

    # ---- requests ---------------------------------------------------------------
    def submit(self, prompt_ids: Sequence[int], options: Optional[GenerateOptions] = None) -> RequestHandle:
        vocab = self.model.spec.vocab_size
        for t in prompt_ids:
            if not 0 <= int(t) < vocab:
                raise InfernumError(f"token id {t} is outside the vocabulary of {vocab}")
        seq = self.scheduler.add_request(prompt_ids, options or GenerateOptions())
        handle = RequestHandle(seq)
        self._handles[seq.id] = handle
        return handle

    def cancel(self, handle: RequestHandle) -> None:
        self.scheduler.cancel(handle.seq)

    def has_work(self) -> bool:
        # (a step launched ahead is taken back by the next ``step`` even if its requests have all ended)
        return self.scheduler.has_work() or (self._ahead is not None and self._ahead[2])

    # ---- one iteration -------------------------------------------------------------
    def step(self) -> List[Tuple[RequestHandle, GenerationEvent]]:
        """One scheduling round and one model step; returns the new events."""
        t0 = time.perf_counter()
        prepared, in_flight = None, False
        if self._ahead is not None:
            plan, prepared, in_flight = self._ahead
            self._ahead = None
            if in_flight:
                # It runs already, on the tokens the step before it selected.  Requests that
                # ended meanwhile (end-of-sequence, cancel) computed one token in vain, which
                # is dropped below; one that arrived waits for the next step.
                self.stats.ahead_used += 1
                self.stats.ahead_launched += 1
            elif self.scheduler.ahead_still_holds(plan):
                self.stats.ahead_used += 1
            else:
                self.stats.ahead_voided += 1
                plan, prepared = None, None
        else:
            plan = None
        if plan is None:
            plan = self.scheduler.schedule()
        self.stats.preemptions = self.scheduler.num_preemptions
        events: List[Tuple[RequestHandle, GenerationEvent]] = []
        if plan.portions:
            wanting = [p for p in plan.portions if p.wants_logits]
            choices = []
            for p in wanting:
                sp = p.seq.options.sampling
                choices.append(None if sp is None else
                               (sp, len(p.seq.generated_ids), recent_window(p.seq.tokens, sp)))
            caches = [p.seq.cache for p in plan.portions]
            decode_only = in_flight or (self.decoder is not None and all(
                p.count == 1 and p.wants_logits for p in plan.portions) and self.decoder.can_take(caches))
            riding = None if decode_only else self._portion_beside_decodes(plan)
            if in_flight:
                chosen = True
            elif riding is not None:
                # decoded tokens (there may be none) and one prompt portion: recorded per (bucket
                # of the batch, bucket of the portion's rows)
                decodes = [p for p in plan.portions if p is not riding]
                caches = [p.seq.cache for p in decodes]
                wanting = decodes + ([riding] if riding.wants_logits else [])
                # (`choices` is in the order of `wanting`: the decoded tokens, then the portion's last row)
                width = self._recent_width(choices)
                sample = pack_choices(choices, width) if width else None
                prc = riding.seq.cache
                prepared = self.decoder.prepare(caches, width, portion=(prc, riding.count, riding.wants_logits))
                chosen = self.decoder.launch(prepared, caches, [p.seq.token_at(p.start) for p in decodes], sample,
                                             portion=(prc, riding.tokens))
                self.h2d_bytes += 4 * int(prepared.ints.numel())
                logits = self.decoder.last.logits
                decode_only = True  # the result comes back the same way
            elif decode_only:
                width = self._recent_width(choices)
                sample = pack_choices(choices, width) if width else None
                if prepared is None or prepared.prepared_for != tuple(rc.request_id for rc in caches) \
                        or (prepared.recent.shape[1] if prepared.recent is not None else 0) != width:
                    prepared = self.decoder.prepare(caches, width)
                chosen = self.decoder.launch(prepared, caches,
                                             [p.seq.token_at(p.start) for p in plan.portions], sample)
                self.h2d_bytes += 16 * len(plan.portions)
                logits = self.decoder.last.logits
            else:
                entries = [StepEntry(p.seq.cache, p.tokens, [p.count - 1] if p.wants_logits else [])
                           for p in plan.portions]
                logits = self.runner.step(entries)
                self.h2d_bytes += self.runner.last_upload_bytes
                chosen = self.sampler.select(logits, choices) if logits is not None and wanting else None
            self.scheduler.commit(plan)
            # (after a step launched ahead in which a request turned out to have ended, the
            # next step comes from the scheduler, which takes that request's pages back)
            if decode_only and not (in_flight and any(p.seq.finished for p in plan.portions)):
                # While this step runs: plan the next one and fill in all of it but the
                # tokens, so that little is left to do between the two steps.
                ahead = self.scheduler.plan_decode_ahead()
                if ahead is not None:
                    nxt = [p.seq.cache for p in ahead.portions]
                    width = self._recent_width([p.seq.options.sampling and (p.seq.options.sampling, 0, ())
                                                for p in ahead.portions])
                    ready = self.decoder.prepare(nxt, width) if self.decoder.can_take(nxt) else None
                    launched = ready is not None and riding is None and self._launch_ahead(plan, ahead, ready, nxt)
                    self._ahead = (ahead, ready, launched)
            if chosen is not None:
                t_wait = time.perf_counter()
                if decode_only:
                    with_portion = riding is not None and riding.wants_logits
                    picked, flags = self.decoder.read_result(len(wanting) - (1 if with_portion else 0), with_portion)
                else:
                    host = torch.cat([chosen, self.runner.rt.err]).cpu().tolist()
                    picked, flags = host[:-1], host[-1]
                self.stats.wait_seconds += time.perf_counter() - t_wait
                self.d2h_bytes += 4 * (len(picked) + 1)
                if flags:
                    self.runner.check_errors()
                for p, tok in zip(wanting, picked):
                    handle = self._handles.get(p.seq.id)
                    if handle is None or p.seq.finished:
                        continue  # it ended while this step, launched ahead, ran
                    emitted = self.scheduler.append_token(p.seq, tok)
                    if emitted is not None:
                        self.stats.generated_tokens += 1
                        ev = GenerationEvent("token", token=emitted)
                        handle.events.append(ev)
                        events.append((handle, ev))
            for p in plan.portions:
                if p.count == 1 and p.start >= len(p.seq.prompt_ids):
                    self.stats.decode_tokens += 1
                else:
                    self.stats.prefill_tokens += p.count
            self.stats.steps += 1
        for handle in list(self._handles.values()):
            if handle.seq.finished and not handle._reported_finish:
                handle._reported_finish = True
                if handle.seq.finish_reason == FinishReason.ERROR:
                    ev = GenerationEvent("error", message=handle.seq.error)
                else:
                    ev = GenerationEvent("finished", reason=handle.seq.finish_reason)
                handle.events.append(ev)
                events.append((handle, ev))
                del self._handles[handle.id]
        self.stats.step_seconds += time.perf_counter() - t0
        return events

    def _launch_ahead(self, plan: StepPlan, ahead: StepPlan, ready, caches) -> bool:
        """Launches the planned next decode step now, behind the one in flight, fed
        on the device with the tokens that one selects: the host then reads a step's
        tokens while the next step runs, and the GPU does not wait for the host
        between the two.  Possible when the rows are those of the step in flight,
        in its order, and no row's sampling needs the tokens not yet seen (a
        repetition penalty looks at the most recent ones)."""
        if not self.config.launch_ahead or self.decoder.last is None or self.decoder.last.portion:
            return False
        if [p.seq.id for p in ahead.portions] != [p.seq.id for p in plan.portions]:
            return False
        choices = []
        for p in ahead.portions:
            sp = p.seq.options.sampling
            if sp is not None and sp.repetition_penalty != 1.0:
                return False
            # (the token of the step in flight is not appended yet: this will be the one after it)
            choices.append(None if sp is None else (sp, len(p.seq.generated_ids) + 1, ()))
        width = self._recent_width(choices)
        sample = pack_choices(choices, width) if width else None
        self.decoder.launch(ready, caches, None, sample, feed_from=self.decoder.last)
        self.h2d_bytes += 12 * len(caches)
        return True

    @staticmethod
    def _recent_width(choices) -> int:
        """0 when every row of ``choices`` is greedy; else the width of the recorded
        step's recent-token buffer: the largest repetition-penalty window among the
        rows that have a penalty, rounded up (``DecodeRunner.recent_width``).  The
        window is a property of the request, so the width does not change while the
        same requests decode."""
        rows = [c[0] for c in choices if c]
        if not rows:
            return 0
        return DecodeRunner.recent_width([sp.repetition_penalty_window for sp in rows
                                          if sp.repetition_penalty != 1.0])

    GRAPH_PORTION_MIN = 16

    def _portion_beside_decodes(self, plan: StepPlan):
        """The step's one prompt portion if the step is "decoded tokens (or none),
        then one prompt portion": such steps recur - while a long prompt is fed in
        portions beside the decoding requests, and for every prompt that comes
        alone - so they are run from recorded graphs like steps of decoded tokens
        alone, one recording per bucket of the portion's length (a shorter portion
        is followed by rows that belong to no request).  A portion that does not
        end its prompt is cut by a few rows where that makes the rows of the
        recorded step (decoded tokens rounded up to their bucket, plus the portion)
        a multiple of the prompt kernels' tile."""
        if self.decoder is None or not plan.portions:
            return None
        *decodes, last = plan.portions
        if last.count < self.GRAPH_PORTION_MIN or (last.count == 1 and last.wants_logits) \
                or not all(p.count == 1 and p.wants_logits for p in decodes):
            return None
        m = self.config.token_multiple
        if m > 0 and not last.wants_logits:
            rows = bucket_for(len(decodes)) + last.count
            extra = rows % m
            if extra and extra * 16 <= rows and last.count - extra >= self.GRAPH_PORTION_MIN:
                last.count -= extra  # its pages stay held for the next step
        if not self.decoder.can_take([p.seq.cache for p in decodes], (last.seq.cache, last.count, last.wants_logits)):
            return None
        return last

    def run_until_done(self, handles: Optional[Sequence[RequestHandle]] = None) -> None:
        while self.has_work() and (handles is None or any(not h.finished for h in handles)):
            self.step()
        self._take_back_ahead()
        self.scheduler._reap()

    def _take_back_ahead(self) -> None:
        """A step launched ahead for requests that have all ended meanwhile is read and dropped."""
        while self._ahead is not None and self._ahead[2] and not self.scheduler.has_work():
            self.step()

    # ---- the reference's entry points ------------------------------------------------
    def generate(self, prompt_ids: Sequence[int], options: Optional[GenerateOptions] = None) -> List[int]:
        """Prompt token ids in, generated token ids out."""
        handle = self.submit(prompt_ids, options)
        self.run_until_done([handle])
        if handle.seq.finish_reason == FinishReason.ERROR:
            raise InfernumError(handle.seq.error or "generation failed")
        return handle.tokens

    def generate_stream(self, prompt_ids: Sequence[int],
                        options: Optional[GenerateOptions] = None) -> Iterator[int]:
        handle = self.submit(prompt_ids, options)
        while not handle.finished:
            for h, ev in self.step():
                if h is handle and ev.kind == "token":
                    yield ev.token
                elif h is handle and ev.kind == "error":
                    raise InfernumError(ev.message or "generation failed")
        self._take_back_ahead()
        self.scheduler._reap()

    def generate_batch(self, prompts: Sequence[Sequence[int]],
                       options=None) -> List[List[int]]:
        """Several requests at once through continuous batching; ``options``
        is one GenerateOptions for all or a list with one per prompt."""
        if options is None or isinstance(options, GenerateOptions):
            options = [options] * len(prompts)
        handles = [self.submit(p, o) for p, o in zip(prompts, options)]
        self.run_until_done(handles)
        for h in handles:
            if h.seq.finish_reason == FinishReason.ERROR:
                raise InfernumError(h.seq.error or "generation failed")
        return [h.tokens for h in handles]
