"""The sequence cache: slots, paged keys and values per group of layers, and
fixed-size per-sequence state.

A *slot* is one live sequence.  Keys and values live in *groups*: layers whose
mixers ask for the same thing (kv heads, key and value size, window) share one pool of
pages ``[layer, page, kv_head, position_in_page, head_dim]`` with a page list
per slot; groups with other needs have a pool of their own.  A group with a
window gives back the pages that no later query can see.  Pages and slots
return to their pools when a sequence is closed and are handed out again.

Beside the keys and values every layer may own a tensor of fixed size per slot
(``StateRequest``), zeroed when a slot is opened; this architecture asks for
none, recurrent or convolutional mixers would.

The reference's Llama path has one growing cache per layer and a single offset
(src/model.h:78-87, src/model.cpp:569-574); slots exist only in its batched GLM
path, as rows of batch arrays that are re-packed on join and leave
(src/glm5_forward.cpp:327-395).  Nothing is re-packed here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import KVRequest, StateRequest
from .pages import CacheError, CacheFull, PagePool, SlotTable

PAGE_SIZE = 64


@dataclass
class KVLayerView:
    """What a mixer sees of the cache during one step."""
    k: torch.Tensor               # [pages, kv_heads, page_size, head_dim] of this layer
    v: torch.Tensor               # [pages, kv_heads, page_size, value_dim or head_dim]
    block_table: torch.Tensor     # int32 [batch rows, pages per row] for this step; -1: no page
    page_size: int
    owns: bool                    # False: the layer reads another layer's keys and values


class KVGroup:
    def __init__(self, request: KVRequest, n_pages: int, page_size: int):
        self.request = request
        self.page_size = page_size
        self.pool = PagePool(n_pages)
        self.owners: List[int] = []                    # schedule entries with storage here
        self.pages: Dict[int, List[int]] = {}          # slot -> physical page per logical page (-1: given back)
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None
        self._k_store: Optional[torch.Tensor] = None
        self._v_store: Optional[torch.Tensor] = None

    def allocate(self, dtype: torch.dtype, device) -> None:
        r = self.request
        # one page more than the pool hands out: rows that only pad a batch write there
        shape = (len(self.owners), self.pool.n_pages + 1, r.kv_heads, self.page_size)
        self.k, self._k_store = self._guarded(shape + (r.head_dim,), dtype, device)
        self.v, self._v_store = self._guarded(shape + (r.value_dim or r.head_dim,), dtype, device)

    GUARD = 512                    # elements of a known pattern before and after each pool
    PATTERN = 1.5

    @classmethod
    def _guarded(cls, shape, dtype, device):
        """A zeroed tensor of ``shape`` inside a larger allocation whose first and last ``GUARD`` elements hold a
        pattern: a kernel that writes before or beyond the pool (a page number out of range) changes them, and
        ``guards_intact`` says so."""
        n = 1
        for d in shape:
            n *= d
        store = torch.zeros(n + 2 * cls.GUARD, dtype=dtype, device=device)
        store[:cls.GUARD] = cls.PATTERN
        store[-cls.GUARD:] = cls.PATTERN
        return store[cls.GUARD:cls.GUARD + n].view(shape), store

    def guards_intact(self) -> bool:
        for store in (self._k_store, self._v_store):
            if store is None:
                continue
            edge = torch.cat([store[:self.GUARD], store[-self.GUARD:]])
            if not bool((edge == self.PATTERN).all()):
                return False
        return True

    def bytes_per_token(self, itemsize: int) -> int:
        r = self.request
        return len(self.owners) * r.kv_heads * (r.head_dim + (r.value_dim or r.head_dim)) * itemsize

    def first_needed_page(self, length: int) -> int:
        """Logical pages below this hold no key that a query at position
        ``length`` or later can see."""
        w = self.request.window
        if w <= 0:
            return 0
        return max(0, length - w + 1) // self.page_size


class SequenceCache:
    """Slots, key/value groups and per-sequence state for one model.

    ``requests[i]`` is what schedule entry ``i`` asks for: a ``KVRequest`` or
    None, a ``StateRequest`` or None, and the entry whose keys and values it
    reads instead of its own (or None)."""

    def __init__(self, requests: Sequence[Tuple[Optional[KVRequest], Optional[StateRequest], Optional[int]]],
                 max_tokens: int, dtype: torch.dtype = torch.bfloat16, device="cpu",
                 page_size: int = PAGE_SIZE, max_slots: Optional[int] = None, allocate: bool = True):
        if max_tokens < 1:
            raise CacheError(f"max_tokens must be positive, got {max_tokens}")
        self.page_size = page_size
        self.n_pages = (max_tokens + page_size - 1) // page_size
        self.max_tokens = self.n_pages * page_size
        self.dtype = dtype
        self.device = device
        self.slots = SlotTable(max_slots if max_slots else min(self.n_pages, 65536))
        self.lengths: Dict[int, int] = {}
        self.groups: List[KVGroup] = []
        self.entry_group: List[Optional[Tuple[int, int]]] = []   # schedule entry -> (group, layer in group)
        self.entry_owns: List[bool] = []
        by_key: Dict[KVRequest, int] = {}
        for i, (kv, _state, src) in enumerate(requests):
            if src is not None:
                if not 0 <= src < i or self.entry_group[src] is None or not self.entry_owns[src]:
                    raise CacheError(f"schedule entry {i} reads the cache of entry {src}, which owns none")
                if kv is not None:
                    src_req = self.groups[self.entry_group[src][0]].request
                    if (kv.kv_heads, kv.head_dim, kv.value_dim or kv.head_dim) != (
                            src_req.kv_heads, src_req.head_dim, src_req.value_dim or src_req.head_dim):
                        raise CacheError(f"schedule entry {i} cannot read entry {src}'s cache: head shapes differ")
                    # the owner gives back the pages its own window no longer reaches: a reader that looks
                    # further back would find them gone (the kernels skip pages that are not there)
                    if src_req.window > 0 and not 0 < kv.window <= src_req.window:
                        raise CacheError(f"schedule entry {i} (window {kv.window or 'none'}) cannot read entry "
                                         f"{src}'s cache, which keeps only a window of {src_req.window}")
                self.entry_group.append(self.entry_group[src])
                self.entry_owns.append(False)
                continue
            if kv is None:
                self.entry_group.append(None)
                self.entry_owns.append(False)
                continue
            if kv not in by_key:
                by_key[kv] = len(self.groups)
                self.groups.append(KVGroup(kv, self.n_pages, page_size))
            g = self.groups[by_key[kv]]
            self.entry_group.append((by_key[kv], len(g.owners)))
            self.entry_owns.append(True)
            g.owners.append(i)
        self.state: Dict[int, torch.Tensor] = {}
        self._state_requests = {i: s for i, (_kv, s, _src) in enumerate(requests) if s is not None}
        if allocate:
            for g in self.groups:
                g.allocate(dtype, device)
            for i, s in self._state_requests.items():
                # one row more than there are slots, for rows that only pad a batch
                self.state[i] = torch.zeros((self.slots.n_slots + 1, *s.shape), dtype=s.dtype, device=device)

    @property
    def pad_page(self) -> int:
        """A page no sequence owns; padding rows of a batch write and read it."""
        return self.n_pages

    @property
    def pad_slot(self) -> int:
        return self.slots.n_slots

    # -- slots ---------------------------------------------------------------
    def open(self) -> int:
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        for g in self.groups:
            g.pages[slot] = []
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        self.slots.free(slot)                           # raises if the slot is not live
        for g in self.groups:
            g.pool.free(p for p in g.pages.pop(slot) if p >= 0)
        del self.lengths[slot]

    def length(self, slot: int) -> int:
        if not self.slots.is_live(slot):
            raise CacheError(f"slot {slot} is not live")
        return self.lengths[slot]

    # -- growth --------------------------------------------------------------
    def reserve(self, wanted: Dict[int, int]) -> None:
        """Makes room for each slot to reach its new length.  Either every
        slot gets its pages or none does (``CacheFull``)."""
        plan: List[Tuple[KVGroup, int, int]] = []
        for g in self.groups:
            need = 0
            for slot, new_len in wanted.items():
                if not self.slots.is_live(slot):
                    raise CacheError(f"slot {slot} is not live")
                if new_len < self.lengths[slot]:
                    raise CacheError(f"slot {slot} cannot shrink from {self.lengths[slot]} to {new_len}")
                n = (new_len + self.page_size - 1) // self.page_size - len(g.pages[slot])
                if n > 0:
                    plan.append((g, slot, n))
                    need += n
            if need > g.pool.n_free:
                raise CacheFull(f"cache is full: {need} more pages of {self.page_size} tokens wanted, "
                                f"{g.pool.n_free} of {g.pool.n_pages} free")
        for g, slot, n in plan:
            g.pages[slot].extend(g.pool.alloc(n))

    def commit(self, slot: int, new_len: int) -> bool:
        """Records the new length and gives back pages that fell out of a
        window; returns whether any page was given back."""
        self.lengths[slot] = new_len
        any_gone = False
        for g in self.groups:
            first = g.first_needed_page(new_len)
            pages = g.pages[slot]
            gone = [p for p in pages[:first] if p >= 0]
            if gone:
                g.pool.free(gone)
                for i in range(min(first, len(pages))):
                    pages[i] = -1
                any_gone = True
        return any_gone

    def gives_back_at(self, length: int) -> bool:
        """Whether a sequence that has just reached ``length`` has a page to give back that it still needed
        at ``length - 1`` (only groups with a window ever do)."""
        return any(g.first_needed_page(length) != g.first_needed_page(length - 1) for g in self.groups)

    def truncate(self, slot: int, new_len: int) -> None:
        """Forgets the positions from ``new_len`` on (the reference's
        ``KVCache::trim``, src/model.cpp:630-650).  Positional caches shrink
        for free; a group that already gave back pages inside the kept range,
        or a layer with fixed-size state, cannot be rewound."""
        cur = self.length(slot)
        if not 0 <= new_len <= cur:
            raise CacheError(f"cannot truncate slot {slot} of length {cur} to {new_len}")
        if self._state_requests and new_len != cur:
            raise CacheError("sequences with fixed-size state cannot be rewound")
        keep = (new_len + self.page_size - 1) // self.page_size
        for g in self.groups:
            if any(p < 0 for p in g.pages[slot][g.first_needed_page(new_len):keep]):
                raise CacheError("a windowed group already gave back pages needed at that length")
        for g in self.groups:
            pages = g.pages[slot]
            g.pool.free(p for p in pages[keep:] if p >= 0)
            del pages[keep:]
        self.lengths[slot] = new_len

    # -- views ---------------------------------------------------------------
    def block_tables(self, slots: Sequence[int], device=None, width: Optional[int] = None) -> List[List[List[int]]]:
        """Per group, per batch row, the physical page of every logical page
        (padded with -1 to a common width)."""
        out = []
        for g in self.groups:
            rows = [g.pages[s] for s in slots]
            w = max([len(r) for r in rows] + [1]) if width is None else width
            out.append([r + [-1] * (w - len(r)) for r in rows])
        return out

    def view(self, entry: int, block_tables: Sequence[torch.Tensor]) -> Optional[KVLayerView]:
        loc = self.entry_group[entry]
        if loc is None:
            return None
        gi, li = loc
        g = self.groups[gi]
        return KVLayerView(g.k[li], g.v[li], block_tables[gi], self.page_size, self.entry_owns[entry])

    def state_of(self, entry: int) -> Optional[torch.Tensor]:
        return self.state.get(entry)

    # -- accounting ----------------------------------------------------------
    def tokens_held(self) -> int:
        """Tokens held by live sequences, each rounded up to whole pages."""
        return sum((n + self.page_size - 1) // self.page_size * self.page_size for n in self.lengths.values())

    def check_guards(self) -> None:
        """Raises if anything was written before or beyond a pool of keys or values (reads the guard words from
        the device: it waits for the work launched so far)."""
        for i, g in enumerate(self.groups):
            if not g.guards_intact():
                raise CacheError(f"the guard words around the key/value pool of cache group {i} were overwritten")

    def check(self) -> None:
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            held = [p for pages in g.pages.values() for p in pages if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError("a page is held by two sequences")
            if len(held) != g.pool.n_held:
                raise CacheError("a page is held by no sequence")
            if set(g.pages) != set(self.slots.live()):
                raise CacheError("page lists and live slots differ")
