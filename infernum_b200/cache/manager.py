"""The cache manager: pages of keys and values with a block table per request,
grouped by what layers need, and slots of fixed-size per-request state.

* A *group* is a set of scheduled layer runs with the same paged-cache needs
  (kv heads, head size, window).  Each group has its own page pool, its own
  device pools (one K and one V tensor ``[pages, kv_heads, page_size, hd]``
  per member) and its own block table per request; one page id covers all
  members of its group.  The reference has a single implicit group: one table
  indexes every layer (infernum-cuda/src/inner/cuda/paged_kv_cache.rs:45-112,
  719-721).
* Pages are taken per step for exactly the tokens of that step (``extend``),
  counted as cached after the step ran (``commit``), and given back when the
  request ends (``release``) or - in a group with a window - once every token
  on them is out of reach of all later queries.  A returned page is handed out
  again first.  (The reference allocates a whole prompt at admission and
  frees only at the end: infernum-runtime/src/scheduler.rs:289-337.)
* A request also holds one *slot* while it lives: the index of its row in
  every state tensor ``[slots, *shape]`` that a mixer declared; the row is
  zeroed when the slot is taken.

All bookkeeping is host-side and runs without a GPU (``device=None``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..errors import CacheError, OutOfPagesError
from ..parts.base import PagedCacheSpec, StateSpec
from .pages import PagePool


@dataclass
class LayerCache:
    """What a mixer gets for one scheduled run."""

    group: int = -1  # index into StepContext.block_tables; -1: no paged cache
    k_pool: Optional[torch.Tensor] = None
    v_pool: Optional[torch.Tensor] = None
    page_size: int = 0
    num_pages: int = 0
    state: Optional[torch.Tensor] = None  # [slots, *shape]
    owner: bool = True  # False: this run reads another run's cache and must not write


@dataclass
class CacheGroup:
    spec: PagedCacheSpec
    positions: List[int]  # schedule positions that own a cache in this group
    pool: PagePool


@dataclass
class RequestCache:
    """Everything the manager holds for one live request."""

    request_id: object
    slot: int
    num_tokens: int = 0  # tokens whose keys/values are in the cache
    reserved_tokens: int = 0  # tokens that pages are held for (>= num_tokens)
    tables: List[List[int]] = field(default_factory=list)  # per group; -1 = given back
    released: bool = False
    serial: int = 0  # which admission this is: a request that comes back after preemption gets a new one
    version: int = 0  # counts changes of the tables (the manager bumps it)
    _arrays: Optional[tuple] = None  # (version, the tables as int32 arrays)

    def table_arrays(self):
        """The block tables as numpy int32 arrays, rebuilt only after a change
        (a step copies them into its upload buffer)."""
        import numpy as np

        if self._arrays is None or self._arrays[0] != self.version:
            self._arrays = (self.version, [np.asarray(t, dtype=np.int32) for t in self.tables])
        return self._arrays[1]


class CacheManager:
    def __init__(self, needs: Sequence, page_size: int, num_pages, max_requests: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, memory_fraction: float = 0.9):
        """``needs``: one item per schedule position with attributes
        ``paged`` (PagedCacheSpec or None), ``state`` (StateSpec or None) and
        ``cache_of`` (an earlier position or None).  ``num_pages`` sizes the
        groups' pools: one number for all of them, a sequence with one number
        per group (groups are numbered in the order in which the schedule first
        needs them), or a function of the group's ``PagedCacheSpec`` - a group
        whose window lets it give pages back early, or whose keys are small,
        needs fewer or cheaper pages than one that keeps everything.  ``None``:
        as many pages (the same number in every pool) as ``memory_fraction`` of
        the device's free memory holds."""
        if page_size <= 0:
            raise CacheError("page_size must be positive")
        if max_requests <= 0:
            raise CacheError("max_requests must be positive")
        self.page_size = int(page_size)
        if num_pages is None:
            num_pages = self._pages_that_fit(needs, dtype, device, memory_fraction)
        self._pages_arg = num_pages
        self.group_pages: List[int] = []
        self.max_requests = int(max_requests)
        self.dtype = dtype
        self.device = device
        self.groups: List[CacheGroup] = []
        self.layer_caches: List[LayerCache] = []
        self._free_slots: List[int] = list(range(self.max_requests - 1, -1, -1))
        self._requests: Dict[object, RequestCache] = {}
        self._admissions = 0
        self._state_tensors: List[torch.Tensor] = []
        # One extra slot, and one extra page behind every group's pool (page id
        # num_pages, never handed out), belong to no request: rows that only pad
        # a batch to a fixed size write there.
        self.pad_slot = self.max_requests

        group_of_spec: Dict[PagedCacheSpec, int] = {}
        for need in needs:
            lc = LayerCache()
            if need.cache_of is not None:
                src = self.layer_caches[need.cache_of]
                lc = LayerCache(group=src.group, k_pool=src.k_pool, v_pool=src.v_pool,
                                page_size=src.page_size, num_pages=src.num_pages, owner=False)
            elif need.paged is not None:
                g = group_of_spec.get(need.paged)
                if g is None:
                    g = len(self.groups)
                    group_of_spec[need.paged] = g
                    self.group_pages.append(self._pages_of_group(g, need.paged))
                    self.groups.append(CacheGroup(need.paged, [], PagePool(self.group_pages[g])))
                self.groups[g].positions.append(need.position)
                pages = self.group_pages[g]
                lc.group, lc.page_size, lc.num_pages = g, self.page_size, pages + 1
                if device is not None:
                    shape = (pages + 1, need.paged.kv_heads, self.page_size, need.paged.head_dim)
                    try:
                        lc.k_pool = torch.zeros(shape, dtype=dtype, device=device)
                        lc.v_pool = torch.zeros(shape, dtype=dtype, device=device)
                    except torch.cuda.OutOfMemoryError:
                        el = torch.empty((), dtype=dtype).element_size()
                        per_page = sum(2 * n.paged.kv_heads * self.page_size * n.paged.head_dim * el
                                       for n in needs if n.paged is not None and n.cache_of is None)
                        free = torch.cuda.mem_get_info(device)[0]
                        raise CacheError(
                            f"the cache pools do not fit the device: a page costs {per_page} bytes over all "
                            f"layers, {pages} pages were asked for, {free / 1e9:.1f} GB were free when the "
                            f"pool at schedule position {need.position} could not be made; ask for fewer pages "
                            f"(or num_pages=None for as many as fit)") from None
            if need.state is not None and need.cache_of is None:
                if device is not None:
                    lc.state = torch.zeros((self.max_requests + 1, *need.state.shape),
                                           dtype=need.state.dtype, device=device)
                    self._state_tensors.append(lc.state)
            self.layer_caches.append(lc)

        if not isinstance(self._pages_arg, int) and not callable(self._pages_arg) \
                and len(self._pages_arg) != len(self.groups):
            raise CacheError(f"num_pages names {len(self._pages_arg)} pools, the model has "
                             f"{len(self.groups)} cache groups")

    def _pages_that_fit(self, needs: Sequence, dtype: torch.dtype, device, fraction: float) -> int:
        """Pages per pool so that all pools together take ``fraction`` of the free device memory."""
        if device is None or torch.device(device).type != "cuda":
            raise CacheError("num_pages=None sizes the pools from a CUDA device's free memory: give a device")
        if not 0.0 < fraction <= 1.0:
            raise CacheError("memory_fraction must be in (0, 1]")
        el = torch.empty((), dtype=dtype).element_size()
        per_page = sum(2 * n.paged.kv_heads * self.page_size * n.paged.head_dim * el
                       for n in needs if n.paged is not None and n.cache_of is None)
        if per_page == 0:
            return 1
        free = torch.cuda.mem_get_info(device)[0]
        pages = int(fraction * free // per_page) - 1  # (a page behind every pool is kept for padding rows)
        if pages < 1:
            raise CacheError(f"no room for cache pages: a page costs {per_page} bytes, {free} are free")
        return pages

    def _pages_of_group(self, g: int, spec: PagedCacheSpec) -> int:
        arg = self._pages_arg
        if callable(arg):
            n = arg(spec)
        elif isinstance(arg, int):
            n = arg
        else:
            if g >= len(arg):
                raise CacheError(f"num_pages names {len(arg)} pools, the model has more cache groups")
            n = arg[g]
        if int(n) <= 0:
            raise CacheError(f"cache group {g}: a pool needs at least one page, got {n}")
        return int(n)

    # ---- sizes --------------------------------------------------------------
    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    @property
    def num_pages(self) -> int:
        """The size of the smallest pool (all pools, when one number sized them)."""
        return min(self.group_pages) if self.group_pages else (
            self._pages_arg if isinstance(self._pages_arg, int) else 0)

    @property
    def pad_page(self) -> int:
        """The page behind the pool that padding rows write to, when every pool
        has the same size (``pad_pages`` gives it per group)."""
        return self.num_pages

    def peak_pages(self, total_tokens: int, step_tokens: int) -> List[int]:
        """Per group, the most pages a request of ``total_tokens`` cached tokens
        holds at any time when it is fed at most ``step_tokens`` a step: all of
        its pages, or, in a group with a window, those the window and one step
        reach (older ones are given back at every commit)."""
        out = []
        for g in self.groups:
            need = self.pages_for(total_tokens)
            if g.spec.window > 0:
                need = min(need, self.pages_for(g.spec.window + step_tokens) + 1)
            out.append(need)
        return out

    def could_ever_hold(self, total_tokens: int, step_tokens: int) -> bool:
        return all(n <= p for n, p in zip(self.peak_pages(total_tokens, step_tokens), self.group_pages))

    def bytes_per_token(self) -> int:
        """Cache bytes one token occupies over all groups and members."""
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * g.spec.kv_heads * g.spec.head_dim * el * len(g.positions) for g in self.groups)

    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def live_requests(self) -> List[RequestCache]:
        return list(self._requests.values())

    def pad_pages(self) -> List[int]:
        """Per group, the page that padding rows write to."""
        return list(self.group_pages)

    # ---- a request's life ---------------------------------------------------
    def admit(self, request_id) -> RequestCache:
        """Takes a slot (zeroing its state rows); no pages yet."""
        if request_id in self._requests:
            raise CacheError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise OutOfPagesError(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        for st in self._state_tensors:
            st[slot].zero_()
        self._admissions += 1
        rc = RequestCache(request_id, slot, tables=[[] for _ in self.groups], serial=self._admissions)
        self._requests[request_id] = rc
        return rc

    def get(self, request_id) -> RequestCache:
        try:
            return self._requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not live") from None

    def has(self, request_id) -> bool:
        return request_id in self._requests

    def pages_needed(self, rc: RequestCache, new_tokens: int) -> List[int]:
        """Per group: pages to add so that ``reserved + new_tokens`` tokens fit."""
        total = self.pages_for(rc.reserved_tokens + new_tokens)
        return [max(0, total - len(t)) for t in rc.tables]

    def can_extend(self, rc: RequestCache, new_tokens: int) -> bool:
        return all(n <= g.pool.num_free for n, g in zip(self.pages_needed(rc, new_tokens), self.groups))

    def extend(self, rc: RequestCache, new_tokens: int) -> None:
        """Holds pages for ``new_tokens`` more tokens, in every group or in none."""
        self._check_live(rc)
        if new_tokens < 0:
            raise CacheError("extend: negative token count")
        need = self.pages_needed(rc, new_tokens)
        for n, g in zip(need, self.groups):
            if n > g.pool.num_free:
                raise OutOfPagesError(
                    f"request {rc.request_id!r} needs {n} more pages, {g.pool.num_free} are free")
        for n, g, table in zip(need, self.groups, rc.tables):
            if n:
                table.extend(g.pool.allocate_many(n))
                rc.version += 1
        rc.reserved_tokens += new_tokens

    def commit(self, rc: RequestCache, new_tokens: int) -> None:
        """The step ran: ``new_tokens`` more tokens are cached.  Pages of a
        windowed group that no later query can reach are given back."""
        self._check_live(rc)
        if rc.num_tokens + new_tokens > rc.reserved_tokens:
            raise CacheError("commit: more tokens than pages were held for")
        rc.num_tokens += new_tokens
        for g, table in zip(self.groups, rc.tables):
            w = g.spec.window
            if w <= 0:
                continue
            # the next query sits at position >= num_tokens and reads keys
            # >= num_tokens - w + 1; page i holds [i*ps, (i+1)*ps)
            first_needed = rc.num_tokens - w + 1
            i = 0
            while i < len(table) and (i + 1) * self.page_size <= first_needed:
                if table[i] >= 0:
                    g.pool.free(table[i])
                    table[i] = -1
                    rc.version += 1
                i += 1

    def cancel_reservation(self, rc: RequestCache) -> None:
        """Gives back pages held beyond the cached tokens (a step that did not run)."""
        self._check_live(rc)
        keep = self.pages_for(rc.num_tokens)
        for g, table in zip(self.groups, rc.tables):
            while len(table) > keep:
                page = table.pop()
                if page >= 0:
                    g.pool.free(page)
        rc.reserved_tokens = rc.num_tokens
        rc.version += 1

    def release(self, rc: RequestCache) -> None:
        """The request ended (or is preempted): pages and slot go back."""
        self._check_live(rc)
        for g, table in zip(self.groups, rc.tables):
            for page in table:
                if page >= 0:
                    g.pool.free(page)
            table.clear()
        self._free_slots.append(rc.slot)
        rc.released = True
        rc.version += 1
        rc.num_tokens = rc.reserved_tokens = 0
        del self._requests[rc.request_id]

    def _check_live(self, rc: RequestCache) -> None:
        if rc.released or self._requests.get(rc.request_id) is not rc:
            raise CacheError(f"request {rc.request_id!r} is not live (released twice?)")

    # ---- invariants, for tests ----------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held."""
        for gi, g in enumerate(self.groups):
            held: Dict[int, object] = {}
            for rc in self._requests.values():
                for page in rc.tables[gi]:
                    if page < 0:
                        continue
                    if page in held:
                        raise CacheError(f"group {gi}: page {page} is held by "
                                         f"{held[page]!r} and {rc.request_id!r}")
                    held[page] = rc.request_id
                    if not g.pool.is_in_use(page):
                        raise CacheError(f"group {gi}: page {page} is held but marked free")
            if len(held) != g.pool.num_used:
                raise CacheError(f"group {gi}: {g.pool.num_used} pages are out, "
                                 f"{len(held)} are in tables (a page was lost)")
        slots = [rc.slot for rc in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a request slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a request slot was lost")
