"""One step's worth of tokens, packed, with the index arrays the kernels read.

Sequences of a step are laid one after another: ``token_ids[T]`` with, per
token, its batch row ``tok_seq`` and absolute position ``tok_pos``.  All index
arrays are built on the host as one int32 buffer and reach the device in one
copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


QUERY_TILES = (128,)        # queries per block of the tensor-core prefill attention


class Workspace:
    """Scratch memory for kernels, owned by the engine and grown on demand.

    ``keep_outgrown``: a buffer that became too small stays alive beside its larger successor.  Recorded CUDA
    graphs hold the address of the buffer they were recorded with, so a workspace that graphs use must never
    free one (a decode runner records a graph per context bucket, and a later bucket may need more scratch
    than an earlier one)."""

    def __init__(self, device, keep_outgrown: bool = False):
        self.device = device
        self.keep_outgrown = keep_outgrown
        self._buf: Optional[torch.Tensor] = None
        self._outgrown: List[torch.Tensor] = []

    def floats(self, n: int) -> torch.Tensor:
        # zeroed when made: the attention kernel keeps counters in it that must start at zero
        # (and returns them to zero itself)
        if self._buf is None or self._buf.numel() < n:
            if self._buf is not None and self.keep_outgrown:
                self._outgrown.append(self._buf)
            self._buf = torch.zeros(max(n, 1 << 16), dtype=torch.float32, device=self.device)
        return self._buf

    def reserve(self, n: int) -> None:
        self.floats(n)


@dataclass
class StepBatch:
    n_tokens: int
    n_rows: int
    token_ids: torch.Tensor           # int32 [T]
    tok_pos: torch.Tensor             # int32 [T] absolute position of each token
    tok_seq: torch.Tensor             # int32 [T] batch row of each token
    slot_ids: torch.Tensor            # int32 [B] cache slot of each batch row
    row_start: torch.Tensor           # int32 [B + 1] first packed token of each row
    row_pos0: torch.Tensor            # int32 [B] position of each row's first token in this step
    want_rows: Optional[torch.Tensor]  # int32 [R] packed indices whose logits are wanted
    n_wanted: int
    block_tables: List[torch.Tensor]  # per cache group: int32 [B, pages]
    max_kv_len: int                   # longest sequence after this step
    max_new: int                      # most tokens any row brings
    workspace: Workspace
    # per tile size (128 queries): (int32 [tiles] batch row, int32 [tiles] first new token, count)
    tiles: Dict[int, Tuple[torch.Tensor, torch.Tensor, int]] = field(default_factory=dict)
    # per tile size, on the host and in the tiles' order: the position after each tile's last query (the keys its
    # queries may see when no window cuts them)
    tile_keys: Dict[int, List[int]] = field(default_factory=dict)
    host_slots: List[int] = field(default_factory=list)
    host_new: List[int] = field(default_factory=list)
    # what a part has worked out for this step and wants to find again in the next layer (keyed as it likes)
    memo: Dict[Any, Any] = field(default_factory=dict)

    @property
    def is_decode(self) -> bool:
        return self.max_new == 1


def pack_step(slots: Sequence[int], starts: Sequence[int], tokens: Sequence[Sequence[int]],
              want: Sequence[Sequence[int]], tables: List[List[List[int]]], workspace: Workspace,
              device) -> StepBatch:
    """Builds the device-side index arrays of a step.  ``starts[i]`` is the
    length of row i before the step, ``want[i]`` lists the places among its
    new tokens whose logits are wanted."""
    B = len(slots)
    counts = [len(t) for t in tokens]
    T = sum(counts)
    row_start = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(counts, out=row_start[1:])
    tok = np.concatenate([np.asarray(t, dtype=np.int64) for t in tokens]) if T else np.zeros(0, np.int64)
    seq = np.repeat(np.arange(B, dtype=np.int64), counts)
    pos = np.arange(T, dtype=np.int64) - np.repeat(row_start[:-1], counts) + np.repeat(
        np.asarray(starts, dtype=np.int64), counts)
    wanted = [int(row_start[i]) + int(w) for i in range(B) for w in want[i]]
    pieces = [tok, pos, seq, np.asarray(slots, np.int64), row_start, np.asarray(starts, np.int64),
              np.asarray(wanted, np.int64)]
    tile_counts = []
    tile_keys = {}
    for size in QUERY_TILES:
        # the tiles with the most keys to visit come first: the attention kernels start them first, so
        # that the long ones do not run alone at the end
        order = sorted(((starts[i] + min(a + size, counts[i]), i, a) for i in range(B) for a in range(0, counts[i], size)),
                       key=lambda x: -x[0])
        tile_rows = [i for _, i, _ in order]
        tile_first = [a for _, _, a in order]
        pieces += [np.asarray(tile_rows, np.int64), np.asarray(tile_first, np.int64)]
        tile_counts.append(len(tile_rows))
        tile_keys[size] = [k for k, _, _ in order]
    n_fixed = len(pieces)
    widths = []
    for g in tables:
        arr = np.asarray(g, dtype=np.int64).reshape(B, -1)
        widths.append(arr.shape[1])
        pieces.append(arr.reshape(-1))
    # pad every piece to a multiple of 4 ints so each view starts 16-byte aligned
    offsets, total = [], 0
    for p in pieces:
        offsets.append(total)
        total += (p.size + 3) // 4 * 4
    host = np.zeros(max(total, 4), dtype=np.int32)
    for p, o in zip(pieces, offsets):
        host[o:o + p.size] = p
    dev = torch.from_numpy(host).pin_memory().to(device, non_blocking=True) if str(device) != "cpu" \
        else torch.from_numpy(host)

    def view(i: int) -> torch.Tensor:
        return dev[offsets[i]:offsets[i] + pieces[i].size]

    bts = [view(n_fixed + gi).view(B, widths[gi]) for gi in range(len(tables))]
    tiles = {size: (view(7 + 2 * i), view(8 + 2 * i), tile_counts[i]) for i, size in enumerate(QUERY_TILES)}
    return StepBatch(
        n_tokens=T, n_rows=B, token_ids=view(0), tok_pos=view(1), tok_seq=view(2), slot_ids=view(3),
        row_start=view(4), row_pos0=view(5), want_rows=view(6) if wanted else None, n_wanted=len(wanted),
        block_tables=bts, max_kv_len=max([s + c for s, c in zip(starts, counts)] + [0]),
        max_new=max(counts + [0]), workspace=workspace, tiles=tiles, tile_keys=tile_keys, host_slots=list(slots),
        host_new=counts)
