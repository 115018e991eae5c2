"""Decode steps from fixed device buffers, recorded once as CUDA graphs.

A step in which every request brings exactly one token has the same sequence
of kernel launches whatever the requests are; only numbers change: tokens,
positions, cache lengths, slots and block tables.  A ``DecodeRunner`` keeps
those in fixed device buffers per *batch bucket* (the batch size rounded up to
1, 2, 4, 8, 16, 24, 32, 48, 64, ...), fills them from the host each step, pads
the bucket with rows that belong to no request (they write to a page and a
state slot reserved for padding), and replays the graph recorded for that
bucket.  Requests may come and go between steps without a new recording; a
graph is recorded per (bucket, cache-length class, width of the sampling rows), the first
time it is needed, after one eager step.

A step of decoded tokens and a few prompt portions (the steps that recur while
prompts are fed in portions - one portion, or the end of one prompt and the
start of the next - and every step of a prompt that is alone) is recorded the
same way, per bucket of the portions' rows together (``portion_bucket``): the
recorded step has 1, 3 or 12 entries for portions (``portion_entries``), of which a step may
leave some empty, followed by an entry that belongs to no request and takes the
rows left over (it attends to, and writes, the page reserved for padding), so
that portions of any lengths up to the bucket replay one recording.  What
differs from step to step - which rows belong to which portion, where their
last rows are - is data in the device buffers, not shape.

Three ways to feed it:
  * from the host (``Engine``): tokens, positions and lengths are copied from
    pinned memory every step, changed block-table rows too;
  * from the step before (``launch(feed_from=...)``): positions, lengths and
    tables come from the host as above, the tokens are the ones the step
    launched before selects, copied on the device, so the step can be launched
    while that one still runs and the host reads its tokens meanwhile;
  * from the device (``pin``): a fixed set of requests whose tokens are the ones
    the previous step selected and whose positions advance on the device; the
    host only reserves pages ahead and uploads the tables once.  Nothing is read
    back between steps.

The reference records a graph for batch size one only, with six stable device
buffers (infernum-cuda/src/inner/cuda_graph_engine.rs:970-1133); larger batches
rebuild and run eagerly every step (:1549-1598).
"""

from __future__ import annotations

import collections
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import RequestCache
from ..ops import core
from ..errors import CacheError
from .step import ModelRunner, StepContext

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)


def bucket_for(n: int) -> int:
    if n <= 0:
        return 0  # (a prompt portion alone: no row for a decoded token)
    for b in BUCKETS:
        if n <= b:
            return b
    return -(-n // 128) * 128


def portion_bucket(n: int) -> int:
    """Rows a recorded step holds for a prompt portion of ``n`` rows: multiples of
    16 up to 64, of 64 beyond.  A portion cut at ``max_prefill_tokens`` fills its
    bucket; only the last portion of a prompt leaves rows over, 32 on average."""
    step = 16 if n <= 64 else 64
    return -(-n // step) * step


@dataclass
class _Slot:
    """Buffers and graph of one (bucket, cache-length class, sampling, feed) key."""

    size: int
    ints: torch.Tensor  # device [6, size]: tokens, positions, kv_len, slot ids, token sources, recent places
    host_ints: torch.Tensor  # pinned mirror
    tables: torch.Tensor  # device [groups, size, MB]
    host_tables: torch.Tensor  # pinned mirror
    selected: torch.Tensor  # device [size] int32
    ctx: StepContext
    rows: List[Optional[Tuple[object, List[int]]]] = field(default_factory=list)  # who sits where
    host_np: object = None  # host_ints' memory as a numpy array (cheap to fill from lists)
    host_tables_np: object = None  # the same for host_tables
    rows_written: List[bool] = field(default_factory=list)  # a row that pads the bucket is written once
    portion: int = 0  # rows held for the prompt portions that ride along (0: decoded tokens only)
    entries_k: int = 0  # entries held for them
    uploaded: Optional[torch.cuda.Event] = None  # after the last upload from the pinned mirrors
    prepared_for: Optional[tuple] = None  # request ids a prepared, not yet launched step is for
    result: Optional[torch.Tensor] = None  # device [size + 1]: the selected tokens, then the error word
    host_results: Optional[list] = None  # two pinned mirrors, used in turn
    result_events: Optional[list] = None  # and the events after their copies
    result_turn: int = 0
    sampled: Optional[torch.Tensor] = None
    params: Optional[torch.Tensor] = None
    host_params: Optional[torch.Tensor] = None
    recent: Optional[torch.Tensor] = None
    host_recent: Optional[torch.Tensor] = None
    mask: Optional[torch.Tensor] = None
    host_mask: Optional[torch.Tensor] = None
    graph: Optional[torch.cuda.CUDAGraph] = None
    logits: Optional[torch.Tensor] = None
    eager_steps: int = 0
    launches_per_step: int = 0


class DecodeRunner:
    # The recent tokens of a sampling row (for its repetition penalty) sit in a fixed buffer
    # [rows, width]; the width is the largest window among the step's rows rounded up to a
    # multiple of this, and part of the key a step is recorded under, so that a window of
    # any length is seen whole.
    RECENT_WIDTH = 64

    @classmethod
    def recent_width(cls, windows) -> int:
        """Buffer width for sampling rows whose repetition-penalty windows are ``windows``."""
        w = max(list(windows) + [1])
        return -(-w // cls.RECENT_WIDTH) * cls.RECENT_WIDTH
    # Buffers and graphs are kept for this many (bucket, cache-length class, sampling, feed,
    # portion) keys; beyond it the one unused for longest is dropped (a graph holds its own
    # activations: some 65 KB a row at the 8B layer sizes, 35 MB for a portion of 512).
    MAX_RECORDED = 256
    # Entries a recorded step may hold for prompt portions: the smallest of these that takes the
    # step's portions (a step with more runs kernel by kernel).  Part of a recording's key.
    PORTION_ENTRIES = (1, 3, 12)

    @classmethod
    def portion_entries(cls, n: int) -> Optional[int]:
        return next((k for k in cls.PORTION_ENTRIES if n <= k), None)

    def __init__(self, runner: ModelRunner, max_model_len: int, use_graph: bool = True):
        self.runner = runner
        self.cache = runner.cache
        self.model = runner.model
        self.rt = runner.rt
        self.use_graph = use_graph
        self.MB = max(1, self.cache.pages_for(max_model_len))
        self.max_model_len = int(max_model_len)
        self._slots: Dict[tuple, _Slot] = {}
        self._pinned: Optional[Tuple[tuple, List[RequestCache]]] = None
        self.last: Optional[_Slot] = None
        # results of launched steps on their way to the host, oldest first
        self._reads: collections.deque = collections.deque(maxlen=4)
        # how the steps so far ran: kernel by kernel, recorded (and replayed at once), replayed
        self.counts = {"eager": 0, "recorded": 0, "replayed": 0, "dropped": 0}

    # ---- buffers -------------------------------------------------------------------
    def _slot(self, key: tuple) -> _Slot:
        slot = self._slots.get(key)
        if slot is not None:
            self._slots[key] = self._slots.pop(key)  # most recently used last
            return slot
        while len(self._slots) >= self.MAX_RECORDED:
            pinned = self._pinned[0] if self._pinned else None
            victim = next((k for k, v in self._slots.items() if k != pinned and v is not self.last), None)
            if victim is None:
                break
            del self._slots[victim]
            self.counts["dropped"] += 1
        size, kv_cap, sampling, _feed, portion, K = key
        dev = self.rt.device
        G = len(self.cache.groups)
        arange = torch.arange(size + 1, dtype=torch.int32, device=dev)
        if portion == 0:
            # (row 4: for a step launched behind another, which of that step's selected tokens
            # each row takes as its input; -1 for a token that comes from the host.  Row 5: where
            # in the row's recent tokens that token goes too, or -1)
            ints = torch.zeros((6, size), dtype=torch.int32, device=dev)
            host_ints = torch.zeros((6, size), dtype=torch.int32).pin_memory()
            host_ints[4:] = -1
            tables = torch.full((G, size, self.MB), -1, dtype=torch.int32, device=dev)
            ctx = StepContext(
                n_rows=size, n_entries=size, token_ids=ints[0], positions=ints[1], row_entry=arange[:size],
                cu_rows=arange, q_start=ints[1], kv_len=ints[2], slot_ids=ints[3], logit_rows=arange[:size],
                block_tables=[tables[g] for g in range(G)], host_cu_rows=list(range(size + 1)),
                host_kv_len=[], max_rows_per_entry=1, max_kv_len=kv_cap, all_decode=True)
            # (how a mixer spreads these rows over its kernels is the mixer's to decide: it sees
            # one row per entry and the longest cache the recorded step may meet, ``max_kv_len``,
            # and keeps its plan in ``ctx.scratch``, which lives as long as the recording)
        else:
            # `size` decoded tokens (one row and one entry each), then the entries of the prompt
            # portions with up to `portion` rows together, then an entry of the rows left over,
            # which belongs to no request.  One flat buffer holds all that changes from step to
            # step: tokens | positions | row_entry (a row each) | cu_rows (entries + 1) |
            # q_start | kv_len | slots (an entry each) | logit rows (decoded rows and the last
            # row of every portion) | token sources of the decoded rows (size; see above).
            rows, entries = size + portion, size + K + 1
            offs = self._portion_offsets(size, portion, K)
            ints = torch.zeros(offs["end"], dtype=torch.int32, device=dev)
            host_ints = torch.zeros(offs["end"], dtype=torch.int32).pin_memory()
            tables = torch.full((G, entries, self.MB), -1, dtype=torch.int32, device=dev)
            view = lambda name, n: ints[offs[name]: offs[name] + n]  # noqa: E731
            ctx = StepContext(
                n_rows=rows, n_entries=entries, token_ids=view("tok", rows), positions=view("pos", rows),
                row_entry=view("rowe", rows), cu_rows=view("cu", entries + 1), q_start=view("q0", entries),
                kv_len=view("kv", entries), slot_ids=view("sl", entries),
                # (a portion's last row is always a logit row: a row more through the head
                # costs nothing, and a step whose portion ends its prompt needs no recording of its own)
                logit_rows=view("logit", size + K),
                block_tables=[tables[g] for g in range(G)],
                # (for launch geometry: one portion at its longest, the entries behind it empty)
                host_cu_rows=list(range(size + 1)) + [rows] * (K + 1), host_kv_len=[], max_rows_per_entry=portion,
                max_kv_len=kv_cap, all_decode=False)
        n_sel = size + K   # rows whose token is selected
        slot = _Slot(size=size, ints=ints, host_ints=host_ints, tables=tables,
                     host_tables=torch.full(tuple(tables.shape), -1, dtype=torch.int32).pin_memory(),
                     selected=torch.zeros(n_sel, dtype=torch.int32, device=dev), ctx=ctx,
                     rows=[None] * tables.shape[1], rows_written=[False] * tables.shape[1], portion=portion,
                     entries_k=K)
        slot.host_np = slot.host_ints.numpy()
        slot.result = torch.zeros(n_sel + 1, dtype=torch.int32, device=dev)
        slot.host_results = [torch.zeros(n_sel + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
        slot.result_events = [torch.cuda.Event(), torch.cuda.Event()]
        if sampling:
            f = core.SAMPLE_PARAM_FLOATS
            slot.sampled = torch.zeros(n_sel, dtype=torch.int32, device=dev)
            slot.params = torch.zeros((n_sel, f), dtype=torch.float32, device=dev)
            slot.host_params = torch.zeros((n_sel, f), dtype=torch.float32).pin_memory()
            slot.recent = torch.zeros((n_sel, int(sampling)), dtype=torch.int32, device=dev)
            slot.host_recent = torch.zeros((n_sel, int(sampling)), dtype=torch.int32).pin_memory()
            slot.mask = torch.zeros(n_sel, dtype=torch.bool, device=dev)
            slot.host_mask = torch.zeros(n_sel, dtype=torch.bool).pin_memory()
        self._slots[key] = slot
        return slot

    @staticmethod
    def _portion_offsets(size: int, portion: int, K: int) -> Dict[str, int]:
        """Where the parts of a portion step's flat int32 buffer begin (``K`` entries for portions)."""
        rows, entries = size + portion, size + K + 1
        offs, at = {}, 0
        for name, n in (("tok", rows), ("pos", rows), ("rowe", rows), ("cu", entries + 1), ("q0", entries),
                        ("kv", entries), ("sl", entries), ("logit", size + K), ("src", size), ("rpos", size)):
            offs[name] = at
            at += n
        offs["end"] = at
        return offs

    def _fill_tables(self, slot: _Slot, caches: Sequence[RequestCache]) -> bool:
        """Brings the host mirror of the block tables up to date; True if it changed.
        A row is rewritten when another request (or another admission of the same
        request) sits in it, or when its request's tables changed since the row
        was last written (the cache manager counts those changes)."""
        changed = False
        if slot.host_tables_np is None:
            slot.host_tables_np = slot.host_tables.numpy()
        tab = slot.host_tables_np
        pads = self.cache.pad_pages()
        for r in range(len(slot.rows)):
            rc = caches[r] if r < len(caches) else None
            seen = (rc.request_id, rc.serial, rc.version) if rc is not None else None
            if slot.rows[r] == seen and (seen is not None or slot.rows_written[r]):
                continue
            slot.rows[r] = seen
            slot.rows_written[r] = True
            changed = True
            tab[:, r, :] = -1
            if rc is None:
                # a row that pads a batch sits at position 0; the entry behind a prompt portion
                # has up to a bucket of rows: every page of its table is the page kept for padding
                for g in range(len(self.cache.groups)):
                    if slot.portion and r == len(slot.rows) - 1:
                        tab[g, r, :] = pads[g]
                    else:
                        tab[g, r, 0] = pads[g]
                continue
            for g, t in enumerate(rc.table_arrays()):
                n = min(len(t), self.MB)
                tab[g, r, :n] = t[:n]
        return changed

    # ---- the recorded body -----------------------------------------------------------
    def _body(self, slot: _Slot, device_feed: bool) -> None:
        slot.logits = self.model.forward(slot.ctx, self.cache.layer_caches)
        core.argmax(slot.logits, slot.selected)
        if slot.sampled is not None:
            core.sample(slot.logits, slot.params, slot.recent, slot.sampled)
            slot.selected.copy_(torch.where(slot.mask, slot.sampled, slot.selected))
        if device_feed:
            core.decode_advance(slot.ctx.token_ids, slot.selected, slot.ctx.positions, slot.ctx.kv_len,
                                slot.ctx.slot_ids, self.cache.pad_slot)
        else:
            # what the host reads after the step, in one piece
            torch.cat((slot.selected, self.rt.err), out=slot.result)

    def _run(self, slot: _Slot, device_feed: bool) -> None:
        if slot.graph is not None:
            slot.graph.replay()
            self.counts["replayed"] += 1
        elif self.use_graph and slot.eager_steps >= 1:
            torch.cuda.synchronize(self.rt.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._body(slot, device_feed)
            slot.graph = graph
            graph.replay()
            self.counts["recorded"] += 1
        else:
            self.counts["eager"] += 1
            before = core.LAUNCHES
            self._body(slot, device_feed)
            slot.launches_per_step = core.LAUNCHES - before
            slot.eager_steps += 1

    def _key(self, caches: Sequence[RequestCache], sampling: int, feed: str, ahead: int = 1,
             portions: Optional[Sequence[Tuple[RequestCache, int, bool]]] = None) -> tuple:
        longest = max([rc.num_tokens for rc in caches] + [0]) + ahead
        for prc, n, _wants in portions or ():
            longest = max(longest, prc.num_tokens + n)
        # cache-length classes: powers of two for decoded tokens alone, of four beside a portion
        # (their kernels' plans depend less on it, and the classes multiply the recordings)
        kv_cap = 256
        while kv_cap < longest:
            kv_cap *= 4 if portions else 2
        # Portions that end their prompts have any length: their rows together are rounded up
        # to a bucket.  When the last one does not end its prompt, the scheduler cut it at
        # ``max_prefill_tokens`` or at the step's budget (less a few rows that make the step's rows
        # a multiple of the prompt kernels' tile): such totals recur and are kept as they are.
        rows = 0
        if portions:
            total = sum(n for _rc, n, _wants in portions)
            rows = portion_bucket(total) if portions[-1][2] else -(-total // 8) * 8
        return (bucket_for(len(caches)), kv_cap, int(sampling), feed, rows,
                self.portion_entries(len(portions)) if portions else 0)

    def can_take(self, caches: Sequence[RequestCache],
                 portions: Optional[Sequence[Tuple[RequestCache, int, bool]]] = None) -> bool:
        if portions is not None and (self.portion_entries(len(portions)) is None or any(
                self.cache.pages_for(prc.num_tokens + n) > self.MB for prc, n, _wants in portions)):
            return False
        return all(self.cache.pages_for(rc.num_tokens + 1) <= self.MB for rc in caches)

    # ---- fed from the host ---------------------------------------------------------------
    def step(self, caches: Sequence[RequestCache], tokens: Sequence[int],
             sample: Optional[tuple] = None) -> torch.Tensor:
        """One decode step of ``caches`` (pages for one more token must be held)
        with the given input tokens.  ``sample``: (params, recent, mask) host
        tensors from ``pack_choices`` when some row samples.  Returns the
        selected token ids, int32 [len(caches)] on the device."""
        width = self.recent_width([sample[1].shape[1]]) if sample is not None else 0
        out = self.launch(self.prepare(caches, width), caches, tokens, sample)
        self._reads.pop()  # the caller reads the device tensor itself
        return out

    def prepare(self, caches: Sequence[RequestCache], sampling: int,
                portions: Optional[Sequence[Tuple[RequestCache, int, bool]]] = None) -> _Slot:
        """The part of a step that does not need the input tokens: picks the
        buffers, fills positions, slots and block tables.  ``sampling``: 0 when
        every row is greedy, else the width of the rows' recent-token buffer
        (``recent_width``).  It may run while the
        step before is still on the GPU (its uploads are waited for first).
        ``portions``: (request, rows, whether its last row's logits are wanted) of
        up to 12 prompt portions (``portion_entries``) that ride along with the decoded
        tokens (there may be none), each continuing its request where the cache
        ends; such a step is recorded per (bucket, bucket of the portions' rows
        together, cache-length class)."""
        B = len(caches)
        slot = self._slot(self._key(caches, sampling, "host", portions=portions))
        if slot.uploaded is not None:
            slot.uploaded.synchronize()  # the pinned mirrors are free to be written again
        pad = slot.size - B
        if portions:
            size, P, K = slot.size, slot.portion, slot.entries_k
            rows, entries = size + P, size + K + 1
            o = self._portion_offsets(size, P, K)
            hn = slot.host_np
            pos, rowe = hn[o["pos"]: o["pos"] + rows], hn[o["rowe"]: o["rowe"] + rows]
            cu, q0 = hn[o["cu"]: o["cu"] + entries + 1], hn[o["q0"]: o["q0"] + entries]
            kv, sl = hn[o["kv"]: o["kv"] + entries], hn[o["sl"]: o["sl"] + entries]
            logit = hn[o["logit"]: o["logit"] + size + K]
            q0[:B] = [rc.num_tokens for rc in caches]
            sl[:B] = [rc.slot for rc in caches]
            if pad:
                hn[o["tok"] + B: o["tok"] + size] = 0
                q0[B:size] = 0
                sl[B:size] = self.cache.pad_slot
            pos[:size] = q0[:size]
            kv[:size] = q0[:size] + 1
            rowe[:size] = range(size)
            cu[: size + 1] = range(size + 1)
            logit[:size] = range(size)
            # the portions' rows one after the other (an entry that is not used has none), then
            # the rows left over, in the entry that belongs to nobody
            at = size
            for j in range(K):
                e = size + j
                if j < len(portions):
                    prc, n, _wants = portions[j]
                    start = prc.num_tokens
                    pos[at: at + n] = range(start, start + n)
                    rowe[at: at + n] = e
                    q0[e], kv[e], sl[e] = start, start + n, prc.slot
                    at += n
                else:
                    q0[e], kv[e], sl[e] = 0, 0, self.cache.pad_slot
                cu[e + 1] = at
                logit[e] = max(at - 1, size)
            left = rows - at
            if left < 0:
                raise CacheError("more portion rows than the recorded step holds")
            pos[at:] = range(left)
            rowe[at:] = size + K
            cu[size + K + 1] = rows
            q0[size + K], kv[size + K], sl[size + K] = 0, left, self.cache.pad_slot
            hn[o["tok"] + at: o["tok"] + rows] = 0
            padded = list(caches) + [None] * pad + [prc for prc, _n, _w in portions] \
                + [None] * (K - len(portions)) + [None]
            if self._fill_tables(slot, padded):
                slot.tables.copy_(slot.host_tables, non_blocking=True)
            slot.prepared_for = tuple(rc.request_id for rc in caches) + tuple(
                (prc.request_id, n) for prc, n, _w in portions)
            return slot
        hn = slot.host_np
        hn[1, :B] = [rc.num_tokens for rc in caches]
        hn[3, :B] = [rc.slot for rc in caches]
        if pad:
            hn[0, B:] = 0
            hn[1, B:] = 0
            hn[3, B:] = self.cache.pad_slot
        hn[2] = hn[1] + 1
        if self._fill_tables(slot, caches):
            slot.tables.copy_(slot.host_tables, non_blocking=True)
        slot.prepared_for = tuple(rc.request_id for rc in caches)
        return slot

    def launch(self, slot: _Slot, caches: Sequence[RequestCache], tokens: Optional[Sequence[int]],
               sample: Optional[tuple] = None,
               portions: Optional[Sequence[Tuple[RequestCache, Sequence[int], bool]]] = None,
               feed_from: Optional[_Slot] = None,
               feed_rows: Optional[Sequence[int]] = None,
               feed_recent: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Uploads the tokens (and sampling rows) and runs the prepared step.
        ``portions``: (request, its tokens of this step, whether its last row's
        token is wanted) for each portion the step was prepared with.
        ``feed_from``: the step takes input tokens from what the step launched
        before it (that slot's, which may be this one) selects, so it can be
        launched while that step still runs, before the host has seen its tokens.
        ``feed_rows`` says which: decoded row ``i`` takes entry ``feed_rows[i]`` of
        that step's selection (its decoded rows in order, then the last rows of its
        prompt portions), or, where that is negative, ``tokens[i]`` from the host;
        without it the rows are those of the step before, in its order, and
        ``tokens`` is not read.  A prompt portion's own tokens always come from the host.
        ``feed_recent[i]``: the place in row ``i``'s recent tokens (``sample``) that the fed
        token takes too, for a row whose repetition penalty must see it; negative for none.
        ``sample``: rows for the decoded tokens in order, then for the portions
        whose token is wanted.
        The step's result starts on its way to the host at once; ``read_result``
        returns the results in the order of the launches."""
        B = len(caches)
        expect = tuple(rc.request_id for rc in caches) + tuple(
            (prc.request_id, len(toks)) for prc, toks, _w in portions or ())
        if slot.prepared_for != expect or bool(slot.portion) != bool(portions):
            raise CacheError("decode step launched for other requests than it was prepared for")
        slot.prepared_for = None
        self.last = slot
        if feed_from is not None and feed_rows is None:
            feed_rows, tokens = range(B), [0] * B
        if portions:
            hn = slot.host_np
            offs = self._portion_offsets(slot.size, slot.portion, slot.entries_k)
            at, rat = offs["src"], offs["rpos"]
            tok_rows, src_rows, rpos_rows = hn[:slot.size], hn[at: at + slot.size], hn[rat: rat + slot.size]
            row = slot.size
            for _prc, toks, _w in portions:
                hn[row: row + len(toks)] = toks
                row += len(toks)
        else:
            tok_rows, src_rows, rpos_rows = slot.host_np[0], slot.host_np[4], slot.host_np[5]
        tok_rows[:B] = tokens
        src_rows[:] = -1
        rpos_rows[:] = -1
        if feed_from is not None:
            src_rows[:B] = feed_rows
            if feed_recent is not None:
                rpos_rows[:B] = feed_recent
        slot.ints.copy_(slot.host_ints, non_blocking=True)
        if sample is not None:
            params, recent, mask = sample
            if slot.recent is None or recent.shape[1] > slot.recent.shape[1]:
                raise CacheError("decode step prepared without room for its rows' recent tokens")
            n_dec = B
            slot.host_params.zero_()
            slot.host_params[:, :3] = 1.0
            slot.host_params[:n_dec] = params[:n_dec]
            slot.host_recent.zero_()
            slot.host_recent[:n_dec, : recent.shape[1]] = recent[:n_dec]
            slot.host_mask.zero_()
            slot.host_mask[:n_dec] = mask[:n_dec]
            k = n_dec
            for j, (_prc, _toks, wants) in enumerate(portions or ()):
                if wants and k < params.shape[0]:
                    slot.host_params[slot.size + j] = params[k]
                    slot.host_recent[slot.size + j, : recent.shape[1]] = recent[k]
                    slot.host_mask[slot.size + j] = mask[k]
                    k += 1
            slot.params.copy_(slot.host_params, non_blocking=True)
            slot.recent.copy_(slot.host_recent, non_blocking=True)
            slot.mask.copy_(slot.host_mask, non_blocking=True)
        if feed_from is not None and B:
            # (behind the uploads: the fed tokens go into the input rows and, where a row's
            # repetition penalty looks at them, into its recent tokens)
            dev_src = slot.ints[at: at + slot.size] if portions else slot.ints[4]
            dev_rpos = slot.ints[rat: rat + slot.size] if portions else slot.ints[5]
            with_recent = feed_recent is not None and sample is not None and slot.recent is not None
            core.feed_tokens(slot.ctx.token_ids[:slot.size], dev_src, feed_from.selected,
                             slot.recent if with_recent else None, dev_rpos if with_recent else None)
        if slot.uploaded is None:
            slot.uploaded = torch.cuda.Event()
        slot.uploaded.record()
        self._run(slot, device_feed=False)
        turn = slot.result_turn
        slot.result_turn ^= 1
        slot.host_results[turn].copy_(slot.result, non_blocking=True)
        slot.result_events[turn].record()
        self._reads.append((slot.host_results[turn], slot.result_events[turn], slot.size,
                            slot.selected.shape[0]))
        for rc in caches:
            self.cache.commit(rc, 1)
        for prc, toks, _w in portions or ():
            self.cache.commit(prc, len(toks))
        self.runner.steps_run += 1
        self.runner.rows_run += B + sum(len(toks) for _prc, toks, _w in portions or ())
        return slot.selected[:B]

    def read_result(self, n: int, portions: Sequence[int] = ()) -> Tuple[List[int], int]:
        """The tokens selected by the oldest launched step not read yet - for its
        first ``n`` decoded tokens and for the last rows of the prompt portions
        ``portions`` (their places among the step's portions) - and the error word
        after them, through pinned memory (this waits for that step, not for one
        launched after it)."""
        buf, event, size, n_sel = self._reads.popleft()
        event.synchronize()
        host = buf.tolist()
        return host[:n] + [host[size + j] for j in portions], host[n_sel]

    # ---- fed from the device ---------------------------------------------------------------
    def pin(self, caches: Sequence[RequestCache], tokens: Sequence[int], steps: int) -> None:
        """Fixes a set of requests for ``steps`` device-fed steps: reserves their
        pages ahead, uploads tokens, positions and tables once."""
        caches = list(caches)
        for rc in caches:
            need = rc.num_tokens + steps - rc.reserved_tokens
            if need > 0:
                self.cache.extend(rc, need)
        key = self._key(caches, False, "device", ahead=steps)
        slot = self._slot(key)
        B = len(caches)
        hi = slot.host_ints
        hi.zero_()
        hi[4:] = -1
        hi[0, :B] = torch.tensor(list(tokens), dtype=torch.int32)
        hi[1, :B] = torch.tensor([rc.num_tokens for rc in caches], dtype=torch.int32)
        hi[3, :B] = torch.tensor([rc.slot for rc in caches], dtype=torch.int32)
        hi[3, B:] = self.cache.pad_slot
        hi[2] = hi[1] + 1
        slot.ints.copy_(hi, non_blocking=True)
        self._fill_tables(slot, caches)
        slot.tables.copy_(slot.host_tables, non_blocking=True)
        torch.cuda.synchronize(self.rt.device)
        self._pinned = (key, caches)
        self.last = slot

    def step_pinned(self) -> torch.Tensor:
        """One step of the pinned requests; nothing crosses the bus."""
        key, caches = self._pinned
        slot = self._slots[key]
        self._run(slot, device_feed=True)
        for rc in caches:
            self.cache.commit(rc, 1)
        self.runner.steps_run += 1
        self.runner.rows_run += len(caches)
        return slot.selected[: len(caches)]
