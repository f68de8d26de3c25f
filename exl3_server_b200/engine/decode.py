"""Decode steps (one token per sequence) from a CUDA graph.

A decode step launches a few hundred small kernels; launched one by one from
Python they take longer to issue than to run.  ``DecodeRunner`` keeps the
step's index arrays in fixed device buffers, records the model's forward pass,
the argmax and the position update into a CUDA graph once, and replays it.
The kernels and the model code are the ones every other step uses; only the
launching differs.

Rows: the runner has a power-of-two number of rows.  Rows without a sequence
are padding: they point at the cache's pad page and pad state row, sit at
position 0 and never advance, and their logits are dropped.  Real rows cannot
see them (a row reads only its own pages), so padding changes no result.

The reference captures nothing (MLX builds a lazy graph per call,
src/model.cpp:594-600); its batched decode step is src/glm5_forward.cpp:397-448.
"""
from __future__ import annotations

import gc
import weakref
from typing import Dict, List, Optional, Sequence

import torch

from ..ops import kernels as K
from .batch import StepBatch, Workspace

SPLIT_BUCKET = 1024       # graphs are recorded for context lengths rounded up to this


def _pow2(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


# Bytes moved between host and device by decode sessions since the process began
# (token ids and page-table rows up, token ids down); the benchmark reads them.
TRANSFERRED = {"h2d": 0, "d2h": 0}


class _Staged:
    """A device buffer with a pinned host copy.  The host copy is rewritten
    only after the previous upload from it has run."""

    def __init__(self, shape, fill: int, device):
        self.dev = torch.full(shape, fill, dtype=torch.int32, device=device)
        self.host = torch.full(shape, fill, dtype=torch.int32).pin_memory()
        self.event: Optional[torch.cuda.Event] = None

    def writable(self) -> torch.Tensor:
        if self.event is not None:
            self.event.synchronize()
        return self.host

    def upload(self) -> None:
        self.dev.copy_(self.host, non_blocking=True)
        TRANSFERRED["h2d"] += self.host.numel() * 4
        if self.event is None:
            self.event = torch.cuda.Event()
        self.event.record()


class DecodeRunner:
    """Fixed buffers and recorded graphs for decode batches of ``rows`` rows
    whose contexts fit ``table_width`` pages."""

    def __init__(self, engine, rows: int, table_width: int):
        self._engine = weakref.ref(engine)              # the engine owns its runners, not the reverse
        self.rows = rows
        self.width = table_width
        dev = engine.device
        cache = engine.cache
        self.token_ids = _Staged((rows,), 0, dev)
        self.tok_pos = _Staged((rows,), 0, dev)
        self.pos_inc = _Staged((rows,), 0, dev)
        self.slot_ids = _Staged((rows,), cache.pad_slot, dev)
        self.tables = [_Staged((rows, table_width), -1, dev) for _ in cache.groups]
        self.tok_seq = torch.arange(rows, dtype=torch.int32, device=dev)
        self.row_start = torch.arange(rows + 1, dtype=torch.int32, device=dev)
        self.next_ids = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.workspace = Workspace(dev, keep_outgrown=True)   # graphs keep the addresses they were recorded with
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_logits: Dict[int, torch.Tensor] = {}
        self.launches: Dict[int, int] = {}
        self.last_bucket = 0
        self.pool = None
        self.holder = None                     # weak reference to the decode session that owns the buffers' contents
        # an all-padding batch of the same shape, for the eager pass before recording
        self.pad_pos = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.pad_slots = torch.full((rows,), cache.pad_slot, dtype=torch.int32, device=dev)
        self.pad_tables = []
        for _ in cache.groups:
            t = torch.full((rows, table_width), -1, dtype=torch.int32, device=dev)
            t[:, 0] = cache.pad_page
            self.pad_tables.append(t)

    @property
    def engine(self):
        eng = self._engine()
        if eng is None:
            raise RuntimeError("decode runner used after its engine was dropped")
        return eng

    def _batch(self, max_kv_len: int, padding: bool) -> StepBatch:
        pos = self.pad_pos if padding else self.tok_pos.dev
        return StepBatch(
            n_tokens=self.rows, n_rows=self.rows, token_ids=self.token_ids.dev, tok_pos=pos,
            tok_seq=self.tok_seq, slot_ids=self.pad_slots if padding else self.slot_ids.dev,
            row_start=self.row_start, row_pos0=pos, want_rows=self.tok_seq, n_wanted=self.rows,
            block_tables=self.pad_tables if padding else [t.dev for t in self.tables],
            max_kv_len=max_kv_len, max_new=1, workspace=self.workspace)

    def _record(self, bucket: int) -> None:
        model, cache = self.engine.model, self.engine.cache
        # One eager pass over an all-padding batch first: it loads every kernel
        # and sizes the scratch memory without touching any sequence.
        torch.cuda.synchronize()
        model.forward(self._batch(bucket, padding=True), cache)
        torch.cuda.synchronize()
        before = K.launch_count()
        g = torch.cuda.CUDAGraph()
        # No garbage collection while the stream is capturing: collecting another
        # CUDA graph there destroys it with calls that are not allowed during a
        # capture, and the capture fails.
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(g, pool=self.pool):
                logits = model.forward(self._batch(bucket, padding=False), cache)
                K.argmax(logits, out=self.next_ids)
                self.token_ids.dev.copy_(self.next_ids)
                self.tok_pos.dev.add_(self.pos_inc.dev)
        finally:
            if gc_was_on:
                gc.enable()
        self.launches[bucket] = K.launch_count() - before
        if self.pool is None:
            self.pool = g.pool()
        self.graphs[bucket] = g
        self.graph_logits[bucket] = logits

    def run(self, max_kv_len: int) -> torch.Tensor:
        """Replays the step for contexts of at most ``max_kv_len`` tokens
        (counted after the step); returns the float32 logits ``[rows, vocab]``,
        valid until the next run."""
        bucket = max(SPLIT_BUCKET, (max_kv_len + SPLIT_BUCKET - 1) // SPLIT_BUCKET * SPLIT_BUCKET)
        if bucket not in self.graphs:
            self._record(bucket)
        self.graphs[bucket].replay()
        self.last_bucket = bucket
        return self.graph_logits[bucket]

    # -- refreshing the buffers ----------------------------------------------
    def _write_pages(self, host_table: torch.Tensor, row: int, pages: List[int]) -> None:
        if len(pages) > self.width:
            raise RuntimeError("decode runner: a sequence outgrew the page table")
        host_table[row, :len(pages)] = torch.as_tensor(pages, dtype=torch.int32)

    def load(self, slots: Sequence[Optional[int]], lengths: Sequence[int], tokens: Optional[Sequence[int]]) -> None:
        """Binds rows 0.. to the given slots at the given lengths (each row's
        next token runs at that position).  Rows beyond the list, and rows
        whose slot is None, pad: pad page, position 0, never advancing."""
        cache = self.engine.cache
        n = len(slots)
        live = [s is not None for s in slots]
        if tokens is not None:
            self.set_tokens(tokens)
        h = self.tok_pos.writable()
        h.zero_()
        h[:n] = torch.as_tensor([int(l) if ok else 0 for l, ok in zip(lengths, live)], dtype=torch.int32)
        self.tok_pos.upload()
        h = self.pos_inc.writable()
        h.zero_()
        h[:n] = torch.as_tensor([1 if ok else 0 for ok in live], dtype=torch.int32)
        self.pos_inc.upload()
        h = self.slot_ids.writable()
        h.fill_(cache.pad_slot)
        h[:n] = torch.as_tensor([s if s is not None else cache.pad_slot for s in slots], dtype=torch.int32)
        self.slot_ids.upload()
        for gi, g in enumerate(cache.groups):
            t = self.tables[gi].writable()
            t.fill_(-1)
            t[:, 0] = cache.pad_page
            for r, s in enumerate(slots):
                if s is not None:
                    t[r, 0] = -1
                    self._write_pages(t, r, g.pages[s])
            self.tables[gi].upload()

    def set_tokens(self, tokens: Sequence[int]) -> None:
        h = self.token_ids.writable()
        h[:len(tokens)] = torch.as_tensor(list(tokens), dtype=torch.int32)
        self.token_ids.upload()

    def push_tables(self, rows_to_slots: Dict[int, int]) -> None:
        """Re-reads the page lists of the given rows from the cache."""
        cache = self.engine.cache
        for gi, g in enumerate(cache.groups):
            t = self.tables[gi].writable()
            for r, s in rows_to_slots.items():
                t[r].fill_(-1)
                self._write_pages(t, r, g.pages[s])
            self.tables[gi].upload()


def runner_for(engine, n_rows: int, max_len: int, holder=None) -> DecodeRunner:
    """One of the engine's runners for at least ``n_rows`` rows and contexts of up to ``max_len`` tokens
    (made on first use, kept for later steps).  A runner's device buffers (positions, slots, page tables,
    tokens) belong to one user at a time: a decode session passes itself as ``holder`` and keeps the runner
    until it is closed or dropped; anyone else gets a runner that no live session holds (a second one of the
    same shape is made when needed) and must be done with it before control returns to the caller."""
    rows = _pow2(max(1, n_rows))
    page = engine.cache.page_size
    width = _pow2(max(16, (max_len + page - 1) // page))
    pool = engine.decode_runners.setdefault((rows, width), [])
    for runner in pool:
        if runner.holder is None or runner.holder() is None or runner.holder() is holder:
            break
    else:
        runner = DecodeRunner(engine, rows, width)
        pool.append(runner)
    runner.holder = weakref.ref(holder) if holder is not None else None
    return runner


class FetchedIds:
    """Token ids on their way to the host; ``get()`` waits for the copy."""

    def __init__(self, host: torch.Tensor, event: torch.cuda.Event, n: int):
        self.host, self.event, self.n = host, event, n

    def get(self) -> List[int]:
        self.event.synchronize()
        return self.host[:self.n].tolist()


class DecodeSession:
    """A fixed set of sequences that advance one token per step.

    ``step(tokens)`` feeds the given token ids (host) or, with ``None``, the
    argmax of the previous step (or what ``feed`` left in its place), which never leaves the device.  Pages are
    reserved as sequences cross page boundaries and the cache's lengths are
    kept in step.  ``fetch_ids()`` starts the copy of the last step's argmax to
    the host, so that the next step can be launched before the host looks at
    it; ``park(rows)`` turns rows whose sequence has ended into padding.
    """

    def __init__(self, engine, slots: Sequence[int], first_tokens: Optional[Sequence[int]], max_new: int = 0):
        self.engine = engine
        self.slots: List[Optional[int]] = list(slots)
        cache = engine.cache
        self.lens = [cache.length(s) for s in self.slots]
        horizon = max(self.lens) + (max_new if max_new > 0 else 4 * SPLIT_BUCKET)
        self.runner = runner_for(engine, len(self.slots), horizon, holder=self)
        self._reserve()
        self.runner.load(self.slots, self.lens, first_tokens)
        self.launches_per_step = 0
        self.closed = False
        self._pinned = [torch.zeros(self.runner.rows, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._fetches = 0

    def _reserve(self) -> Dict[int, int]:
        """Makes sure every live row has a page for its next position; returns
        the rows whose page lists grew."""
        cache = self.engine.cache
        page = cache.page_size
        grew: Dict[int, int] = {}
        want: Dict[int, int] = {}
        for r, s in enumerate(self.slots):
            if s is not None and any(len(g.pages[s]) * page <= self.lens[r] for g in cache.groups):
                want[s] = self.lens[r] + 1
                grew[r] = s
        if want:
            cache.reserve(want)
        return grew

    def step(self, tokens: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Runs one token per sequence; returns the logits ``[n, vocab]`` of
        the sequences (valid until the next step)."""
        if self.closed:
            raise RuntimeError("decode session: step after close")
        cache = self.engine.cache
        page = cache.page_size
        longest = max([n for n, s in zip(self.lens, self.slots) if s is not None] + [0])
        limit = self.engine.model.plan.max_positions
        if limit and longest + 1 > limit:
            from .engine import StepError
            raise StepError(f"decode session: {longest + 1} positions exceed max_position_embeddings {limit}")
        if longest + 1 > self.runner.width * page:
            if tokens is None:
                raise RuntimeError("decode session: contexts outgrew the page table while tokens are fed "
                                   "on the device; give max_new when the session is made")
            self.runner.holder = None
            self.runner = runner_for(self.engine, len(self.slots), longest + 4 * SPLIT_BUCKET, holder=self)
            self._reserve()
            self.runner.load(self.slots, self.lens, None)
        else:
            grew = self._reserve()
            if grew:
                self.runner.push_tables(grew)
        if tokens is not None:
            self.runner.set_tokens(tokens)
        logits = self.runner.run(longest + 1)
        self.launches_per_step = self.runner.launches.get(self.runner.last_bucket, 0)
        shrunk: Dict[int, int] = {}
        for r, s in enumerate(self.slots):
            if s is None:
                continue
            self.lens[r] += 1
            if cache.gives_back_at(self.lens[r]):
                if cache.commit(s, self.lens[r]):          # a windowed group gave a page back
                    shrunk[r] = s
            else:
                cache.lengths[s] = self.lens[r]
        if shrunk:
            self.runner.push_tables(shrunk)
        self.engine.steps_run += 1
        live = [n - 1 for n, s in zip(self.lens, self.slots) if s is not None]
        if live:
            self.engine.count_step(live, [1] * len(live), len(live))
        return logits[:len(self.slots)]

    @property
    def next_ids(self) -> torch.Tensor:
        """The argmax of the last step's logits, on the device."""
        return self.runner.next_ids[:len(self.slots)]

    def feed(self, ids: torch.Tensor) -> None:
        """The next ``step(None)`` runs these token ids (int32 on the device, one per sequence) instead of the
        last step's argmax: tokens sampled on the device go on without a trip to the host."""
        n = len(self.slots)
        self.runner.token_ids.dev[:n].copy_(ids[:n])

    def fetch_ids(self, ids: Optional[torch.Tensor] = None) -> FetchedIds:
        """Starts copying the last step's argmax (or the given ids of that step) to pinned host memory (it must
        be asked for before the next step is launched, which overwrites it)."""
        host = self._pinned[self._fetches % len(self._pinned)]
        self._fetches += 1
        if ids is None:
            host.copy_(self.runner.next_ids, non_blocking=True)
        else:
            host[:ids.numel()].copy_(ids, non_blocking=True)
        TRANSFERRED["d2h"] += host.numel() * 4
        ev = torch.cuda.Event()
        ev.record()
        return FetchedIds(host, ev, len(self.slots))

    def park(self, rows: Sequence[int]) -> None:
        """The sequences of these rows have ended: their rows become padding
        (steps already launched still wrote into their own pages, nothing
        later does).  The cache learns their final lengths."""
        cache = self.engine.cache
        for r in rows:
            s = self.slots[r]
            if s is not None:
                cache.commit(s, self.lens[r])
                self.slots[r] = None
        # positions come from the host's count, which includes the steps in flight
        self.runner.load(self.slots, self.lens, None)

    def close(self) -> None:
        """Records the sequences' lengths in the cache and lets go of the runner."""
        cache = self.engine.cache
        for s, n in zip(self.slots, self.lens):
            if s is not None and cache.slots.is_live(s):
                cache.commit(s, n)
        if self.runner.holder is not None and self.runner.holder() is self:
            self.runner.holder = None
        self.closed = True
