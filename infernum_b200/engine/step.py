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
    """Device-side description of a step, read by every part."""

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

    # ---- building the inputs -------------------------------------------------
    def _build(self, entries: Sequence[StepEntry]) -> StepContext:
        E = len(entries)
        if E == 0:
            raise SchedulingError("a step needs at least one entry")
        if E > self.max_entries:
            raise SchedulingError(f"{E} entries in one step, the limit is {self.max_entries}")
        n_groups = len(self.cache.groups)
        tokens: List[int] = []
        positions: List[int] = []
        row_entry: List[int] = []
        cu_rows = [0]
        q_start, kv_len, slots, logit_rows = [], [], [], []
        for e, ent in enumerate(entries):
            n = len(ent.tokens)
            if n == 0:
                raise SchedulingError(f"entry {e} brings no tokens")
            start = ent.cache.num_tokens
            if ent.cache.reserved_tokens < start + n:
                raise SchedulingError(f"entry {e}: pages are held for {ent.cache.reserved_tokens} "
                                      f"tokens, the step reaches {start + n}")
            for t in ent.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise SchedulingError(f"token id {t} is outside the vocabulary "
                                          f"of {self.vocab_size}")
            base = cu_rows[-1]
            tokens.extend(int(t) for t in ent.tokens)
            positions.extend(range(start, start + n))
            row_entry.extend([e] * n)
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
        tables_flat: List[int] = []
        for g in range(n_groups):
            for ent in entries:
                t = ent.cache.tables[g]
                row = t[:MB] + [-1] * (MB - len(t))
                tables_flat.extend(row)
        R = len(logit_rows)
        pieces = [tokens, positions, row_entry, cu_rows, q_start, kv_len, slots, logit_rows,
                  tables_flat]
        sizes = [len(p) for p in pieces]
        host = torch.tensor([v for p in pieces for v in p], dtype=torch.int32)
        if self.device.type == "cuda":
            host = host.pin_memory()
        dev = host.to(self.device, non_blocking=True)
        self.last_upload_bytes = host.numel() * 4
        views, off = [], 0
        for s in sizes:
            views.append(dev[off: off + s])
            off += s
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
