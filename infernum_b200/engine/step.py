"""The step function: one batch of (request, its next tokens) through the model.

A step may hold any mix of prompt portions and single decoded tokens, cut
anywhere.  Only the tokens it is given are run; everything earlier comes from
the cache.  It returns the logits at the wanted places.

The reference has two separate calls instead - ``forward_prefill`` for one
sequence and ``forward_batch_decode`` for B single tokens
(infernum/src/model.rs:96-132) - and its prefill ignores the start position
(infernum-cuda/src/inner/cuda_graph_engine.rs:1318,1332-1333).  Here a decode
token is simply a portion of length one, and a row at absolute position p of a
request attends to keys 0..p of that request: cached pages plus this step's
own rows, which are written before attention reads them.

Flattened inputs of a step (N rows, E entries), all int32 on the device and
uploaded in one copy from pinned memory:
    token_ids[N], positions[N], row_entry[N], cu_rows[E+1], q_start[E],
    kv_len[E], slot_ids[E], logit_rows[R], block_tables[group][E, MB].
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..errors import InfernumError, KernelError, SchedulingError
from ..ops import core


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens, and the places among
    them (0-based) whose logits are wanted."""

    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepContext:
    """Device-side description of a step, read by every part.

    The tensors are the truth: which rows belong to which entry (``row_entry``,
    ``cu_rows``), where an entry's rows sit in its request (``q_start``,
    ``positions``, ``kv_len``) and which state slot it has (``slot_ids``).  A
    step that is replayed from a recording gets new contents in them each
    time - other requests, portions of other lengths, rows at the end that
    belong to no request - while the host-side fields below stay as they were
    when the step was recorded.  Those describe the step's *shape* and serve
    for launch geometry only: ``n_rows``, ``n_entries``; ``max_rows_per_entry``
    and ``max_kv_len``, upper bounds; ``host_cu_rows``, which in a recorded step
    gives every entry the most rows it may have (not the rows it has);
    ``all_decode``, one row per entry.  ``scratch`` lives as long as the
    recording: a part may keep a plan or a buffer there."""

    n_rows: int
    n_entries: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    row_entry: torch.Tensor
    cu_rows: torch.Tensor
    q_start: torch.Tensor
    kv_len: torch.Tensor
    slot_ids: torch.Tensor
    logit_rows: Optional[torch.Tensor]
    block_tables: List[torch.Tensor]
    # host copies, for launch geometry
    host_cu_rows: List[int] = field(default_factory=list)
    host_kv_len: List[int] = field(default_factory=list)
    max_rows_per_entry: int = 0
    max_kv_len: int = 0
    all_decode: bool = False
    scratch: Dict[str, torch.Tensor] = field(default_factory=dict)


class ModelRunner:
    """Owns the step buffers and runs ``Model.forward`` over the cache."""

    def __init__(self, model, cache: CacheManager, max_rows: int = 8192, max_entries: int = 256):
        self.model = model
        self.cache = cache
        self.rt = model.rt
        self.device = self.rt.device
        self.max_rows = int(max_rows)
        self.max_entries = int(max_entries)
        if self.rt.err is None:
            self.rt.err = core.new_error_word(self.device)
        self.vocab_size = model.spec.vocab_size
        self.steps_run = 0
        self.rows_run = 0
        self.last_upload_bytes = 0
        # pinned staging buffers for the step inputs, used in turn; each carries the
        # event of its last upload, which is waited for before the buffer is written again
        self._staging: List[list] = []
        self._staging_next = 0

    # ---- building the inputs -------------------------------------------------
    STAGING_BUFFERS = 4

    def _upload_buffer(self, n: int):
        """A pinned int32 buffer of at least ``n`` values (tensor and numpy view)
        whose last upload has completed."""
        if len(self._staging) < self.STAGING_BUFFERS:
            self._staging.append([None, None, None])
            self._staging_next = len(self._staging) - 1
        else:
            self._staging_next = (self._staging_next + 1) % self.STAGING_BUFFERS
        slot = self._staging[self._staging_next]
        if slot[2] is not None:
            slot[2].synchronize()
        if slot[0] is None or slot[0].numel() < n:
            t = torch.empty(max(n, 4096) * 2, dtype=torch.int32)
            if self.device.type == "cuda":
                t = t.pin_memory()
            slot[0], slot[1] = t, t.numpy()
        return slot[0], slot[1]

    def _mark_uploaded(self) -> None:
        if self.device.type == "cuda":
            slot = self._staging[self._staging_next]
            if slot[2] is None:
                slot[2] = torch.cuda.Event()
            slot[2].record()

    def _build(self, entries: Sequence[StepEntry]) -> StepContext:
        E = len(entries)
        if E == 0:
            raise SchedulingError("a step needs at least one entry")
        if E > self.max_entries:
            raise SchedulingError(f"{E} entries in one step, the limit is {self.max_entries}")
        n_groups = len(self.cache.groups)
        counts = [len(ent.tokens) for ent in entries]
        cu_rows = [0]
        q_start, kv_len, slots, logit_rows = [], [], [], []
        for e, (ent, n) in enumerate(zip(entries, counts)):
            if n == 0:
                raise SchedulingError(f"entry {e} brings no tokens")
            start = ent.cache.num_tokens
            if ent.cache.reserved_tokens < start + n:
                raise SchedulingError(f"entry {e}: pages are held for {ent.cache.reserved_tokens} "
                                      f"tokens, the step reaches {start + n}")
            base = cu_rows[-1]
            cu_rows.append(base + n)
            q_start.append(start)
            kv_len.append(start + n)
            slots.append(ent.cache.slot)
            for w in ent.want:
                if not 0 <= w < n:
                    raise SchedulingError(f"entry {e}: wanted place {w} is outside its {n} tokens")
                logit_rows.append(base + w)
        N = cu_rows[-1]
        if N > self.max_rows:
            raise SchedulingError(f"{N} tokens in one step, the limit is {self.max_rows}")
        MB = max(1, max(self.cache.pages_for(k) for k in kv_len))
        R = len(logit_rows)
        # one int32 buffer: tokens | positions | row_entry | cu_rows | q_start | kv_len | slots |
        # logit_rows | block tables, filled through numpy in pinned memory and uploaded in one copy
        sizes = [N, N, N, E + 1, E, E, E, R, n_groups * E * MB]
        total = sum(sizes)
        host_t, host = self._upload_buffer(total)
        offs = [0]
        for sz in sizes:
            offs.append(offs[-1] + sz)
        tok = host[offs[0]: offs[1]]
        pos = host[offs[1]: offs[2]]
        rowe = host[offs[2]: offs[3]]
        for e, (ent, n) in enumerate(zip(entries, counts)):
            lo, hi = cu_rows[e], cu_rows[e + 1]
            try:
                tok[lo:hi] = ent.tokens
            except (OverflowError, ValueError, TypeError) as exc:
                raise SchedulingError(f"entry {e}: token ids must be integers inside the vocabulary "
                                      f"of {self.vocab_size} ({exc})") from None
            pos[lo:hi] = np.arange(q_start[e], q_start[e] + n, dtype=np.int32)
            rowe[lo:hi] = e
        if N and (int(tok.min()) < 0 or int(tok.max()) >= self.vocab_size):
            bad = int(tok[(tok < 0) | (tok >= self.vocab_size)][0])
            raise SchedulingError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
        host[offs[3]: offs[4]] = cu_rows
        host[offs[4]: offs[5]] = q_start
        host[offs[5]: offs[6]] = kv_len
        host[offs[6]: offs[7]] = slots
        host[offs[7]: offs[8]] = logit_rows
        tab = host[offs[8]: offs[9]].reshape(n_groups, E, MB) if n_groups else None
        if n_groups:
            tab.fill(-1)
            for e, ent in enumerate(entries):
                for g, t in enumerate(ent.cache.table_arrays()):
                    k = min(len(t), MB)
                    tab[g, e, :k] = t[:k]
        dev = torch.empty(total, dtype=torch.int32, device=self.device)
        dev.copy_(host_t[:total], non_blocking=True)
        self._mark_uploaded()
        self.last_upload_bytes = total * 4
        views = [dev[offs[i]: offs[i + 1]] for i in range(9)]
        tables = [views[8][g * E * MB: (g + 1) * E * MB].view(E, MB) for g in range(n_groups)]
        return StepContext(
            n_rows=N, n_entries=E, token_ids=views[0], positions=views[1], row_entry=views[2],
            cu_rows=views[3], q_start=views[4], kv_len=views[5], slot_ids=views[6],
            logit_rows=views[7] if R else None, block_tables=tables,
            host_cu_rows=cu_rows, host_kv_len=kv_len,
            max_rows_per_entry=max(cu_rows[i + 1] - cu_rows[i] for i in range(E)),
            max_kv_len=max(kv_len), all_decode=(N == E),
        )

    # ---- running ---------------------------------------------------------------
    def reserve(self, entries: Sequence[StepEntry]) -> None:
        """Holds pages for every entry's tokens; on failure nothing stays held."""
        done = []
        try:
            for ent in entries:
                need = ent.cache.num_tokens + len(ent.tokens) - ent.cache.reserved_tokens
                if need > 0:
                    self.cache.extend(ent.cache, need)
                    done.append(ent)
        except InfernumError:
            for ent in done:
                self.cache.cancel_reservation(ent.cache)
            raise

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs one step.  Pages are taken as needed (``OutOfPagesError`` if
        the pool cannot give them; nothing has run then).  Returns float32
        logits [wanted, vocab] on the device in the order of the entries and of
        their ``want`` lists, or None when nothing is wanted."""
        self.reserve(entries)
        ctx = self._build(entries)
        logits = self.model.forward(ctx, self.cache.layer_caches)
        for ent in entries:
            self.cache.commit(ent.cache, len(ent.tokens))
        self.steps_run += 1
        self.rows_run += ctx.n_rows
        return logits

    def check_errors(self) -> None:
        """Reads the device error word (this synchronises) and raises if a
        kernel flagged a bad token, a bad page or a wait that ran out."""
        flags = int(self.rt.err.item())
        if flags:
            self.rt.err.zero_()
            raise KernelError("a kernel reported: " + core.describe_flags(flags))
