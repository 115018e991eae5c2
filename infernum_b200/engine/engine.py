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
from ..ops import core
from ..sampling.params import GenerateOptions
from ..sampling.sampler import Sampler, pack_choices
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
                                  dtype=rt.dtype, device=rt.device, memory_fraction=cfg.cache_memory_fraction)
        self.runner = ModelRunner(model, self.cache, max_rows=cfg.max_tokens_per_step,
                                  max_entries=cfg.max_batch_size)
        max_len = cfg.max_model_len or model.spec.max_position
        self.scheduler = Scheduler(cfg, self.cache, max_len)
        self.sampler = Sampler(rt.device)
        self.stats = EngineStats()
        self._handles: Dict[int, RequestHandle] = {}
        # (in profile mode every operation is launched and timed by itself: no recordings)
        recorded = cfg.cuda_graphs and model.replayable and not core.PROFILE
        self.decoder = DecodeRunner(self.runner, max_len, use_graph=True) if recorded else None
        # the next decode step, planned and prepared while the one before it ran
        # (plan, prepared buffers, whether it is on the GPU already)
        self._ahead: Optional[Tuple[StepPlan, object, bool, object]] = None
        self._flight: Dict[int, int] = {}  # request id -> where the step launched last puts its token
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
        prepared, in_flight, split = None, False, None
        if self._ahead is not None:
            plan, prepared, in_flight, split = self._ahead
            self._ahead = None
            if in_flight:
                # It runs already, on the tokens the step before it selected.  Requests that
                # ended meanwhile (end-of-sequence, cancel) computed one token in vain, which
                # is dropped below; one that arrived waits for the next step.
                self.stats.ahead_used += 1
                self.stats.ahead_launched += 1
            elif self.scheduler.plan_still_holds(plan):
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
            # A step of decoded tokens, alone or beside a few prompt portions, runs from a
            # recording (`split`: its decoded rows and its portions); any other step runs
            # kernel by kernel.
            if not in_flight:
                split = self._recorded_shape(plan)
            if split is not None:
                decodes, riding = split
                wanting = decodes + [p for p in riding if p.wants_logits]
            else:
                wanting = [p for p in plan.portions if p.wants_logits]
            if in_flight:
                chosen = True
            else:
                choices = []
                for p in wanting:
                    sp = p.seq.options.sampling
                    choices.append(None if sp is None else (sp, len(p.seq.generated_ids), self._recent(p.seq, sp)))
                if split is not None:
                    caches = [p.seq.cache for p in decodes]
                    width = self._recent_width(choices)
                    sample = pack_choices(choices, width) if width else None
                    if riding or prepared is None or prepared.prepared_for != tuple(rc.request_id for rc in caches) \
                            or (prepared.recent.shape[1] if prepared.recent is not None else 0) != width:
                        prepared = self.decoder.prepare(
                            caches, width, portions=[(p.seq.cache, p.count, p.wants_logits) for p in riding])
                    chosen = self.decoder.launch(prepared, caches, [p.seq.token_at(p.start) for p in decodes], sample,
                                                 portions=[(p.seq.cache, p.tokens, p.wants_logits) for p in riding])
                    self._note_flight(decodes, riding)
                    self.h2d_bytes += 4 * int(prepared.ints.numel()) if riding else 16 * len(decodes)
                else:
                    entries = [StepEntry(p.seq.cache, p.tokens, [p.count - 1] if p.wants_logits else [])
                               for p in plan.portions]
                    logits = self.runner.step(entries)
                    self.h2d_bytes += self.runner.last_upload_bytes
                    chosen = self.sampler.select(logits, choices) if logits is not None and wanting else None
            self.scheduler.commit(plan)
            if split is not None:
                # While this step runs: schedule the next one as if every request had the token
                # this step selects for it, and launch it behind this one, fed on the device;
                # where that cannot be (it is a step that runs kernel by kernel, or launching
                # ahead is switched off), it is kept and run when the tokens have come.
                ahead = self.scheduler.plan_ahead(plan)
                if ahead is not None:
                    self._ahead = (ahead,) + self._launch_ahead(ahead)
            if chosen is not None:
                t_wait = time.perf_counter()
                if split is not None:
                    picked, flags = self.decoder.read_result(
                        len(decodes), [j for j, p in enumerate(riding) if p.wants_logits])
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
                        p.seq.pending = 0
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

    def _note_flight(self, decodes, riding) -> None:
        """Remembers where the step just launched puts each request's selected token
        (its decoded rows in order, then the last rows of its prompt portions)."""
        self._flight = {p.seq.id: i for i, p in enumerate(decodes)}
        for j, p in enumerate(riding):
            if p.wants_logits:
                self._flight[p.seq.id] = self.decoder.last.size + j

    def _launch_ahead(self, ahead: StepPlan):
        """Launches the planned next step now, behind the one in flight, with the
        tokens that one selects fed on the device: the host then reads a step's
        tokens while the next step runs, and the GPU does not wait for the host
        between the two.  Possible for the steps that run from recordings
        (decoded tokens, with or without prompt portions); a row whose repetition
        penalty looks at the token not yet seen gets it on the device too.  Returns (prepared buffers or None, whether it was launched,
        the step's decoded rows and portions if it runs from a recording)."""
        dec = self.decoder
        split = self._recorded_shape(ahead)
        if split is None:
            return None, False, None
        decodes, riding = split
        caches = [p.seq.cache for p in decodes]
        can_launch = self.config.launch_ahead and dec.last is not None and not any(p.seq.pending for p in riding)
        choices, feed_rows, feed_recent, tokens = [], [], [], []
        for p in decodes + [p for p in riding if p.wants_logits]:
            sp = p.seq.options.sampling
            place = -1
            if sp is None:
                choices.append(None)
            elif p.seq.pending:
                # (the token of the step in flight is not appended yet: this is the one after it;
                # a repetition penalty looks at that token too, so it is given a place at the end
                # of the row's recent tokens, which the device fills in)
                rec = self._recent(p.seq, sp, in_flight=True)
                place = len(rec) - 1
                choices.append((sp, len(p.seq.generated_ids) + 1, rec))
            else:
                choices.append((sp, len(p.seq.generated_ids), self._recent(p.seq, sp)))
            if len(feed_recent) < len(decodes):
                feed_recent.append(place)
        for p in decodes:
            if p.seq.pending:
                feed_rows.append(self._flight.get(p.seq.id, -1))
                tokens.append(0)
                can_launch = can_launch and feed_rows[-1] >= 0
            else:
                feed_rows.append(-1)
                tokens.append(p.seq.token_at(p.start))
        width = self._recent_width(choices)
        if not can_launch:
            return (dec.prepare(caches, width) if not riding else None), False, split
        ready = dec.prepare(caches, width, portions=[(p.seq.cache, p.count, p.wants_logits) for p in riding])
        sample = pack_choices(choices, width) if width else None
        dec.launch(ready, caches, tokens, sample, feed_from=dec.last, feed_rows=feed_rows, feed_recent=feed_recent,
                   portions=[(p.seq.cache, p.tokens, p.wants_logits) for p in riding])
        self._note_flight(decodes, riding)
        self.h2d_bytes += 4 * int(ready.ints.numel())
        return ready, True, split

    @staticmethod
    def _recent(seq: Sequence_, sp, in_flight: bool = False) -> List[int]:
        """The tokens a row's repetition penalty looks at: the last
        ``repetition_penalty_window`` of its request (infernum-runtime/src/engine.rs:508-512);
        none where there is no penalty.  ``in_flight``: the newest token is not known
        yet and gets the last place, which the device fills in."""
        w = sp.repetition_penalty_window
        if sp.repetition_penalty == 1.0 or w <= 0:
            return []
        return seq.last_tokens(w - 1) + [0] if in_flight else seq.last_tokens(w)

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

    # the fewest rows the portions of a recorded step have together (a portion is never cut below it)
    GRAPH_PORTION_MIN = 2

    def _recorded_shape(self, plan: StepPlan):
        """(decoded rows, prompt portions) if the step is one that runs from a
        recording: decoded tokens - or none - beside at most a few prompt portions
        (``DecodeRunner.portion_entries``).  Such steps recur: while long prompts
        are fed in portions beside the decoding requests (one portion, or the end
        of one prompt and the start of the next), and for every prompt that comes
        alone.  They are recorded per bucket of the portions' rows together (rows
        left over belong to no request).  A last portion that does not end its
        prompt is cut by a few rows where that makes the rows of the recorded
        step (decoded tokens rounded up to their bucket, plus the portions) a
        multiple of the prompt kernels' tile.  None for any other step."""
        if self.decoder is None or not plan.portions:
            return None
        decodes = [p for p in plan.portions if p.count == 1 and p.wants_logits]
        riding = [p for p in plan.portions if not (p.count == 1 and p.wants_logits)]
        if not riding:
            return (decodes, riding) if self.decoder.can_take([p.seq.cache for p in decodes]) else None
        if self.decoder.portion_entries(len(riding)) is None \
                or sum(p.count for p in riding) < self.GRAPH_PORTION_MIN:
            return None
        last = riding[-1]
        m = self.config.token_multiple
        if m > 0 and not last.wants_logits:
            rows = bucket_for(len(decodes)) + sum(p.count for p in riding)
            extra = rows % m
            if extra and extra * 16 <= rows and last.count - extra >= self.GRAPH_PORTION_MIN:
                last.count -= extra  # its pages stay held for the next step
        if not self.decoder.can_take([p.seq.cache for p in decodes],
                                     [(p.seq.cache, p.count, p.wants_logits) for p in riding]):
            return None
        return decodes, riding

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
