"""Decoding a fixed set of requests with inputs that live on the device.

While the same requests decode step after step, nothing about a step changes
but the numbers: one token, one position and one cache length per request, and
now and then a new page in a block table.  A ``DecodeSession`` keeps those in
fixed device buffers, so the step - model, token selection, advance - is a
fixed sequence of kernel launches that is recorded once as a CUDA graph and
replayed.  The host still does the page bookkeeping (it knows every position
without asking the device) and copies the block tables when one changed.

The reference does the same for batch size one only: six stable device
buffers and a captured graph (infernum-cuda/src/inner/cuda_graph_engine.rs:970-1133);
larger batches rebuild and run eagerly every step (:1549-1598).
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..cache.manager import RequestCache
from ..ops import core
from ..ops.attention_fast import SM_COUNT_FALLBACK, choose_splits
from .step import ModelRunner, StepContext


class DecodeSession:
    def __init__(self, runner: ModelRunner, caches: Sequence[RequestCache], tokens: Sequence[int],
                 max_steps: int, use_graph: bool = True, sampling_rows: Optional[Sequence[bool]] = None):
        self.runner = runner
        self.cache = runner.cache
        self.model = runner.model
        self.rt = runner.rt
        self.caches = list(caches)
        self.key = tuple(rc.request_id for rc in self.caches)
        dev = self.rt.device
        B = self.B = len(self.caches)
        self.use_graph = use_graph
        self.steps_left = int(max_steps)
        longest = max(rc.num_tokens for rc in self.caches) + max_steps + 1
        self.MB = max(1, self.cache.pages_for(longest))
        n_groups = len(self.cache.groups)

        def i32(values):
            return torch.tensor(list(values), dtype=torch.int32, device=dev)

        self.tokens = i32(tokens)
        self.positions = i32(rc.num_tokens for rc in self.caches)
        self.kv_len = i32(rc.num_tokens + 1 for rc in self.caches)
        self.selected = torch.zeros(B, dtype=torch.int32, device=dev)
        self.host_tokens = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.host_tables = torch.full((n_groups, B, self.MB), -1, dtype=torch.int32).pin_memory()
        self.dev_tables = torch.full((n_groups, B, self.MB), -1, dtype=torch.int32, device=dev)
        self._tables_dirty = True
        self._known_pages = [[0] * n_groups for _ in range(B)]
        self.sampling_rows = list(sampling_rows) if sampling_rows is not None else [False] * B
        self.any_sampling = any(self.sampling_rows)
        if self.any_sampling:
            self.host_params = torch.zeros((B, core.SAMPLE_PARAM_FLOATS), dtype=torch.float32).pin_memory()
            self.dev_params = torch.zeros((B, core.SAMPLE_PARAM_FLOATS), dtype=torch.float32, device=dev)
            self.recent_width = 64
            self.host_recent = torch.zeros((B, self.recent_width), dtype=torch.int32).pin_memory()
            self.dev_recent = torch.zeros((B, self.recent_width), dtype=torch.int32, device=dev)
            self.sample_mask = torch.tensor(self.sampling_rows, dtype=torch.bool, device=dev)
            self.sampled = torch.zeros(B, dtype=torch.int32, device=dev)
        arange = torch.arange(B + 1, dtype=torch.int32, device=dev)
        kv_heads = max([g.spec.kv_heads for g in self.cache.groups] + [1])
        sm = self.rt.options.get("sm_count") or SM_COUNT_FALLBACK
        splits = choose_splits(B, kv_heads, longest, sm)
        self.ctx = StepContext(
            n_rows=B, n_entries=B, token_ids=self.tokens, positions=self.positions,
            row_entry=arange[:B], cu_rows=arange, q_start=self.positions, kv_len=self.kv_len,
            slot_ids=i32(rc.slot for rc in self.caches), logit_rows=arange[:B],
            block_tables=[self.dev_tables[g] for g in range(n_groups)],
            host_cu_rows=list(range(B + 1)), host_kv_len=[], max_rows_per_entry=1,
            max_kv_len=longest, all_decode=True)
        self.ctx.attention_mode = (2, splits)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self._eager_steps = 0
        self.launches_per_step = 0

    # ---- host bookkeeping ---------------------------------------------------------
    def _reserve(self) -> None:
        """Pages for one more token per request; raises OutOfPagesError with
        nothing taken if the pool cannot give them."""
        done = []
        try:
            for rc in self.caches:
                need = rc.num_tokens + 1 - rc.reserved_tokens
                if need > 0:
                    self.cache.extend(rc, need)
                    done.append(rc)
        except Exception:
            for rc in done:
                self.cache.cancel_reservation(rc)
            raise
        for b, rc in enumerate(self.caches):
            for g, table in enumerate(rc.tables):
                if len(table) != self._known_pages[b][g] or self._tables_dirty:
                    n = min(len(table), self.MB)
                    self.host_tables[g, b, :n] = torch.tensor(table[:n], dtype=torch.int32)
                    self._known_pages[b][g] = len(table)
                    self._tables_dirty = True
            # pages a window gave back
            for g, grp in enumerate(self.cache.groups):
                if grp.spec.window > 0:
                    n = min(len(rc.tables[g]), self.MB)
                    self.host_tables[g, b, :n] = torch.tensor(rc.tables[g][:n], dtype=torch.int32)
                    self._tables_dirty = True

    def can_continue(self) -> bool:
        return self.steps_left > 0 and all(
            self.cache.pages_for(rc.num_tokens + 1) <= self.MB for rc in self.caches)

    # ---- the step --------------------------------------------------------------------
    def _body(self) -> None:
        self.logits = self.model.forward(self.ctx, self.cache.layer_caches)
        core.argmax(self.logits, self.selected)
        if self.any_sampling:
            core.sample(self.logits, self.dev_params, self.dev_recent, self.sampled)
            self.selected.copy_(torch.where(self.sample_mask, self.sampled, self.selected))
        core.decode_advance(self.tokens, None if self._feed_host else self.selected,
                            self.positions, self.kv_len)

    def step(self, host_tokens: Optional[Sequence[int]] = None, sample_params=None) -> torch.Tensor:
        """One decode step.  ``host_tokens``: the tokens to feed, copied from
        pinned memory (None: the device feeds itself the tokens it selected).
        Returns the selected token ids, int32 [B] on the device."""
        self._feed_host = host_tokens is not None
        self._reserve()
        if self._tables_dirty:
            self.dev_tables.copy_(self.host_tables, non_blocking=True)
            self._tables_dirty = False
        if host_tokens is not None:
            self.host_tokens.copy_(torch.tensor(list(host_tokens), dtype=torch.int32))
            self.tokens.copy_(self.host_tokens, non_blocking=True)
        if self.any_sampling and sample_params is not None:
            params, recent = sample_params
            self.host_params.copy_(params)
            self.host_recent.zero_()
            self.host_recent[:, : recent.shape[1]] = recent[:, : self.recent_width]
            self.dev_params.copy_(self.host_params, non_blocking=True)
            self.dev_recent.copy_(self.host_recent, non_blocking=True)
        if self.graph is not None and self._graph_feed_host == self._feed_host:
            self.graph.replay()
        elif self.use_graph and self._eager_steps >= 1:
            self._capture()
            self.graph.replay()
        else:
            before = core.LAUNCHES
            self._body()
            self.launches_per_step = core.LAUNCHES - before
            self._eager_steps += 1
        for rc in self.caches:
            self.cache.commit(rc, 1)
        self.steps_left -= 1
        self.runner.steps_run += 1
        self.runner.rows_run += self.B
        return self.selected

    def _capture(self) -> None:
        torch.cuda.synchronize(self.rt.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._body()
        self.graph = graph
        self._graph_feed_host = self._feed_host
