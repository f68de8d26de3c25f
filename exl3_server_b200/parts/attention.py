"""The attention mixer: grouped-query attention over the paged cache.

Per token: ``q, k, v = r Wq^T, r Wk^T, r Wv^T`` (+ biases when the checkpoint
has them, src/model.cpp:558-560, 370-376); heads are contiguous slices of the
projection (``feature = head * head_dim + d``, src/model.cpp:562-564); q and k
get the position encoding; k (rotated) and v go to the cache
(src/model.cpp:566-574); ``o = softmax(q K^T * scale + causal) V`` with query
head h reading kv head ``h // (heads / kv_heads)`` (src/model.cpp:576-578);
``y = concat_h(o) Wo^T`` (src/model.cpp:579-580).  ``window`` > 0 limits a
query at position p to keys ``p - window + 1 .. p``.

The three input projections are one fused matrix, so a step reads ``r`` once.

Which kernels run: prompts in bfloat16 with heads of 64 or 128 go through the tcgen05 attention, after the
position part's own step.  Steps in which every sequence brings one token (decode), in
bfloat16 with heads of 64 or 128, are one kernel: it rotates the queries and the token's own key, takes that key and
value from the projection's output, adds them to the softmax and writes them to the cache (``_decode_fused``;
the position part must offer ``fused_rotation``).  Everything else (float32, other head sizes) takes the
position step and the CUDA-core attention kernel.
"""
from __future__ import annotations

import heapq
import math
import os
from typing import Dict, List, Optional

import numpy as np
import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext, KVRequest, StateRequest
from .linear import Linear
from .registry import position_class, register_mixer
from .spec import MixerSpec, PositionSpec

# Keys per work item of the CUDA-core attention kernel; a multiple of the cache's page size.
SPLIT_KEYS = 256
# Work items (token x kv head x chunk) beyond which the bfloat16 path doubles the chunk length.
BUSY_ITEMS = 1776
# Prompts: the position step inside the q/k/v projection's epilogue where the sizes allow it (0: always a kernel of its own).
PROMPT_FUSED = os.environ.get("EXL3_PROMPT_FUSED", "1") != "0"


class Attention:
    @staticmethod
    def tensor_specs(spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        q, kv = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim
        out = [
            TensorSpec(prefix + "q_proj.weight", (q, spec.width)),
            TensorSpec(prefix + "k_proj.weight", (kv, spec.width)),
            TensorSpec(prefix + "v_proj.weight", (kv, spec.width)),
            TensorSpec(prefix + "o_proj.weight", (spec.width, q)),
        ]
        for name, n in (("q_proj", q), ("k_proj", kv), ("v_proj", kv), ("o_proj", spec.width)):
            out.append(TensorSpec(prefix + name + ".bias", (n,), optional=True, init="zeros"))
        return out

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        if spec.heads < 1 or spec.kv_heads < 1 or spec.heads % spec.kv_heads != 0:
            raise ValueError(f"attention: {spec.heads} heads cannot share {spec.kv_heads} kv heads")
        if spec.head_dim % 16 != 0:
            raise ValueError(f"attention: head_dim must be a multiple of 16, got {spec.head_dim}")
        self.spec = spec
        self.ctx = ctx
        names = ("q_proj", "k_proj", "v_proj")
        w = torch.cat([tensors[prefix + n + ".weight"].to(ctx.dtype) for n in names], dim=0)
        biases = [tensors.get(prefix + n + ".bias") for n in names]
        b = None
        if any(x is not None for x in biases):
            sizes = (spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim, spec.kv_heads * spec.head_dim)
            b = torch.cat([(x.to(ctx.dtype) if x is not None else torch.zeros(n, dtype=ctx.dtype, device=w.device))
                           for x, n in zip(biases, sizes)])
        self.qkv = Linear(w, b, ctx.dtype)
        self.o = Linear(tensors[prefix + "o_proj.weight"], tensors.get(prefix + "o_proj.bias"), ctx.dtype)
        pos = spec.position or PositionSpec(kind="none", dims=0)
        self.position = position_class(pos.kind)(pos, spec.head_dim, ctx)
        self.scale = spec.softmax_scale if spec.softmax_scale is not None else spec.head_dim ** -0.5

    def cache_request(self) -> Optional[KVRequest]:
        return KVRequest(self.spec.kv_heads, self.spec.head_dim, self.spec.window)

    def state_request(self) -> Optional[StateRequest]:
        return None

    takes_then = True       # the last projection may fold its output into the residual (NormAfter)
    takes_raw = True        # the first projection takes a norm's output in two pieces (RawNormed)

    def forward(self, x: torch.Tensor, batch, kv, state, then=None) -> torch.Tensor:
        s = self.spec
        if kv is None:
            raise RuntimeError("attention needs a cache view")
        qkv = self._prompt_fused(x, batch, kv)
        if qkv is not None:
            # prompts: the projection has rotated the queries and put the rotated keys and the values into the
            # cache, from where the attention reads them
            out = torch.empty((qkv.shape[0], s.heads * s.head_dim), dtype=qkv.dtype, device=qkv.device)
            self.attend(qkv, out, batch, kv)
            return self.o(out, then=then)
        qkv = self.qkv(x)
        T = qkv.shape[0]
        out = torch.empty((T, s.heads * s.head_dim), dtype=qkv.dtype, device=qkv.device)
        if not self._decode_fused(qkv, out, batch, kv):
            self.position.rotate_and_store(qkv, batch, kv, s.heads, s.kv_heads, s.head_dim)
            self.attend(qkv, out, batch, kv)
        return self.o(out, then=then)

    def _prompt_fused(self, x, batch, kv):
        """Prompts in bfloat16 with heads and pages of 64, enough rows for the paired GEMM and an attention kernel
        that reads keys and values from the cache only: the q/k/v projection applies the position encoding and
        writes the cache in its epilogue (``Linear.heads_rotated_and_cached``), so the position step is no kernel of
        its own.  None when the step, the sizes or the position part do not allow it."""
        s = self.spec
        fused = getattr(self.position, "fused_rotation", None)
        if batch.max_new <= 1 or fused is None or self.ctx.dtype != torch.bfloat16 or not batch.tiles or not PROMPT_FUSED:
            return None
        if not K.attn_prefill_tc_supported(torch.bfloat16, s.head_dim, kv.page_size):
            return None
        return self.qkv.heads_rotated_and_cached(x, s.heads, s.kv_heads, s.head_dim, kv.page_size, fused(s.head_dim),
                                                 batch, kv)

    def _decode_fused(self, qkv: torch.Tensor, out: torch.Tensor, batch, kv) -> bool:
        """One token per sequence, bfloat16, heads of 64 or 128: the decode kernel rotates the queries and the new key
        itself, takes the token's own key and value from ``qkv`` and writes them to the cache, so the position
        step is no kernel of its own.  False when the step, the sizes or the position part do not allow it."""
        s = self.spec
        fused = getattr(self.position, "fused_rotation", None)
        if batch.max_new != 1 or qkv.dtype != torch.bfloat16 or fused is None:
            return False
        rotation = fused(s.head_dim)
        if rotation is None:
            return False
        inv_freq, rot, pos_scale = rotation
        T = qkv.shape[0]
        if not self._decode_kernel_takes(qkv.dtype, T, kv.page_size):
            return False
        split, head_split, in_block = self._decode_split(T, batch.max_kv_len, kv.page_size, qkv.device)
        head_split, twins = self._decode_twins(head_split, in_block)
        n = self._chunks(batch.max_kv_len, split)
        scratch = None
        if n > 1 and not in_block:
            scratch = batch.workspace.floats(K.attn_tokens_scratch_bytes(T, s.heads, s.head_dim, n) // 4)
        K.attn_decode(qkv, qkv.stride(0), out, kv.k, kv.v, kv.block_table, batch.tok_pos, batch.tok_seq, T,
                      s.heads, s.kv_heads, s.head_dim, kv.page_size, s.window, self.scale, split, n, scratch,
                      inv_freq=inv_freq, rot=rot, pos_scale=pos_scale, write_new=kv.owns, head_split=head_split,
                      in_block=in_block, twins=twins)
        return True

    def _decode_kernel_takes(self, dtype: torch.dtype, T: int, page: int) -> bool:
        """Whether the tensor-core decode kernel takes this mixer's shapes at all (any chunking)."""
        s = self.spec
        return K.attn_decode_supported(dtype, T, s.heads, s.kv_heads, s.head_dim, page, page, 1)

    def attend(self, qkv: torch.Tensor, out: torch.Tensor, batch, kv) -> None:
        s = self.spec
        T = qkv.shape[0]
        if batch.max_new > 1 and batch.tiles and K.attn_prefill_tc_supported(qkv.dtype, s.head_dim, kv.page_size):
            # prompts, heads of 64 or 128: streaming softmax with both products on tcgen05 tensor cores,
            # TMA loads straight from the paged cache, a block per 128 queries
            tile_seq, tile_q0, n_tiles = batch.tiles[128]
            key = ("attn_prefill_variant", s.heads, s.head_dim, s.window)
            variant = batch.memo.get(key)
            if variant is None:
                variant = batch.memo[key] = self._prefill_variant(batch.tile_keys.get(128), kv.page_size, qkv.device)
            K.attn_prefill_tc(qkv, qkv.stride(0), out, kv.k, kv.v, kv.block_table, batch.row_start, batch.row_pos0,
                              tile_seq, tile_q0, n_tiles, s.heads, s.kv_heads, s.head_dim, kv.page_size, s.window,
                              self.scale, variant=variant)
            return
        if self._decode_kernel_takes(qkv.dtype, T, kv.page_size):
            # decoded tokens, heads of 64 or 128: pages by TMA, both products on the tensor cores, a warp per chunk
            split, head_split, in_block = self._decode_split(T, batch.max_kv_len, kv.page_size, qkv.device)
            head_split, twins = self._decode_twins(head_split, in_block)
            n = self._chunks(batch.max_kv_len, split)
            scratch = None
            if n > 1 and not in_block:
                scratch = batch.workspace.floats(K.attn_tokens_scratch_bytes(T, s.heads, s.head_dim, n) // 4)
            K.attn_decode(qkv, qkv.stride(0), out, kv.k, kv.v, kv.block_table, batch.tok_pos, batch.tok_seq, T,
                          s.heads, s.kv_heads, s.head_dim, kv.page_size, s.window, self.scale, split, n, scratch,
                          head_split=head_split, in_block=in_block, twins=twins)
            return
        split = max(SPLIT_KEYS, kv.page_size)
        if split % kv.page_size:
            split = kv.page_size * (split // kv.page_size + 1)
        n = self._chunks(batch.max_kv_len, split)
        # bfloat16 with more work items than the GPU holds at once: chunks twice as long, so that a
        # block's fixed costs are spread over more keys.  float32 keeps one chunking for every
        # batch, so that its results do not depend on the batch at all.
        if qkv.dtype == torch.bfloat16 and T * s.kv_heads * ((batch.max_kv_len + split - 1) // split) > BUSY_ITEMS:
            split *= 2
            n = self._chunks(batch.max_kv_len, split)
        scratch = None
        if n > 1:
            scratch = batch.workspace.floats(K.attn_tokens_scratch_bytes(T, s.heads, s.head_dim, n) // 4)
        K.attn_tokens(qkv, qkv.stride(0), out, kv.k, kv.v, kv.block_table, batch.tok_pos, batch.tok_seq, T,
                      s.heads, s.kv_heads, s.head_dim, kv.page_size, s.window, self.scale, split, n, scratch)

    def _prefill_variant(self, tile_keys, page: int, device: torch.device) -> int:
        """Which form of the tensor-core prompt kernel a step's tiles get (``K.attn_prefill_tc``'s ``variant``): a
        tile a block (1); two tiles a block, the list's first with its last and so on (3); or, for heads of 64, the
        kernel with four blocks an SM (2).  All three are simulated from the list of tiles: a block's time is its
        pages to walk plus three pages' worth for every tile (its start and its end), a page taking 0.9 us on one
        of the two slots an SM has for the first two forms (one slot for heads of 128) and 1.5 us on one of the four
        of the third; the tiles' heads run side by side on as many slots, and a tile goes to the slots that come
        free first, in the list's order.  Constants fitted to thirteen measured workloads (to 9 % in the mean; us
        for forms 1 / 2 / 3, 36 heads of 64 unless said): one prompt of 2,048 tokens 41.9 / 59.1 / 40.2, of 1,536
        28.5 / 39.3 / 34.0, of 8,192 442 / 429 / 455, 24 prompts of 16 to 2,048 tokens 447 / 392 / 470, one of 5,000
        with 16 heads 88.8 / 130 / 130.  The four-block kernel is taken when the better of the others is not
        below 0.93 of it (the model flatters them where tiles are short)."""
        s = self.spec
        if not tile_keys:
            return 0
        sms = K.sm_count(device)
        n = len(tile_keys)
        size = 128
        pages = [((min(k, s.window + size) if s.window > 0 else k) + page - 1) // page for k in tile_keys]
        each = 3                                                # a tile's start and end, in pages

        def makespan(times, slots):
            if len(times) * s.heads <= slots:
                return max(times)
            if len(times) <= 64 and s.heads <= slots:
                # every block on the slot that comes free first: a tile's heads take the slots that are free soonest
                free = np.zeros(slots)
                for t in times:
                    free[np.argpartition(free, s.heads - 1)[:s.heads]] += t
                return float(free.max())
            # many tiles: groups of slots as wide as a tile has heads, what the division leaves over given back as
            # capacity
            groups = slots // s.heads
            if groups == 0:
                return sum(times) * s.heads / slots
            free = [0.0] * groups
            end = 0.0
            for t in times:
                at = heapq.heappop(free) + t
                heapq.heappush(free, at)
                end = max(end, at)
            return max(max(times), end * groups * s.heads / slots)

        slots = sms * (2 if s.head_dim == 64 else 1)
        one = 0.9 * makespan([p + each for p in pages], slots)
        half = (n + 1) // 2
        two = 0.9 * makespan([pages[i] + each + (pages[n - 1 - i] + each if n - 1 - i > i else 0) for i in range(half)],
                             slots)
        best = 3 if two <= one else 1
        if s.head_dim == 64:
            four = 1.5 * makespan([p + each for p in pages], 4 * sms)
            if min(one, two) >= 0.93 * four:
                return 2
        return best

    def _decode_split(self, T: int, max_kv_len: int, page: int, device: torch.device):
        """``(keys per chunk, head_split, in_block)`` (``in_block``: 0, 1 or 2) for the tensor-core decode kernel:
        chunks of whole pages (a power of two of them, at most 64 of 16 KB), into how many groups of work the query
        heads of a kv head are cut
        (``head_split``: that many times the work items, each merge that much smaller, the keys and values read
        again from L2), and whether a block takes a whole (token, group of heads) and merges its up to four chunks in
        shared memory (``in_block``) instead of warps taking equal shares of all chunks and merging through global
        memory.  By a small model of the kernel's time, its constants fitted to a sweep of every chunking at four
        head layouts (36/36 x 64, 16/2 x 64, 32/8 x 128, 32/2 x 128), contexts of 128 to 16,384 tokens and batches of
        1 to 64 (some 5,000 timings; what the model picks is 0.9 % slower in the mean than the best of a case):
        6 us to start; a warp walks its chunk at 0.55 us per 16 KB of keys and values (0.9 us with more than 8 query
        heads in its group: two blocks of instruction columns); when there are more chunks than warps a warp takes
        several in turn; all warps together cannot read faster than the memory does (6.6 TB/s for what is read once,
        12 TB/s from L2 for what the groups of a kv head read again); and the chunks of a (token, group of heads),
        when there is more than one, are merged by a single warp: 3 us, plus per chunk 0.03 us and 0.04 us for every
        head of the group, 2 % more for every group that merges at the same time.  So wide groups of heads in small
        batches are cut into many narrow ones with a fair number of chunks each, one chunk wins for short contexts
        and for batches with a warp's worth of work per sequence (no merge at all), and many short chunks only where
        they are needed to give every SM work.  A block per item costs, for every round of as many blocks as the GPU
        has SMs, 5.5 us and 0.1 us a head of the group (start and the merge in shared memory) and its walk (a
        quarter of the keys per warp), and not less than the memory's time, which its rounds stream some 5 % faster
        at the price of 1 us between rounds; it is taken when that is below 0.95 of the other way's cost: for up to
        about as many items as the GPU has SMs, each too long for one warp, and for several rounds of long items,
        not for many rounds of short ones.  A cluster of two blocks per item (``in_block`` 2: eight warps, five to
        eight chunks, merged by the first block) costs 7 us and 0.1 us a head, an eighth of the keys' walk, and 3 us
        between rounds of half as many clusters as the GPU has SMs: for one sequence of 36 heads at 4,096 tokens
        13.6 us against 14.9 us with a block per item, at 8,192 tokens 19.0 against 23.1; for 8 sequences of 2 kv
        heads with 16 query heads each at 2,048 tokens 14.4 against 16.0.  The choice depends on the step's
        size, not on a token's position: results differ between batch sizes by rounding."""
        s = self.spec
        keys = min(max_kv_len, s.window) if s.window > 0 else max_kv_len
        pages_seq = max(1, (keys + page - 1) // page)
        wide = max(1, s.head_dim // 64)                     # 16 KB stages in a page
        group = s.heads // s.kv_heads
        sms = K.sm_count(device)
        warps = 4 * sms
        best = None                                          # warps share all chunks
        best_blk = None                                      # a block per item
        for head_split in (1, 2, 4, 8, 16):
            if group % head_split:
                continue
            g = group // head_split
            if g > 16:
                continue
            stage_us = 0.55 if g <= 8 else 0.9
            groups = T * s.kv_heads * head_split
            once_us = T * s.kv_heads * pages_seq * wide * 16384 / 6.6e6
            again_us = groups * pages_seq * wide * 16384 / 12.0e6
            per = 1
            while True:
                n = (pages_seq + per - 1) // per
                if n + (1 if s.window > 0 else 0) <= K.ATTN_DECODE_MAX_CHUNKS:     # a window may straddle one chunk more
                    rounds = (groups * n + warps - 1) // warps
                    cost = 6.0 + max(rounds * per * wide * stage_us, once_us, again_us)
                    if n > 1:
                        cost += 3.0 + n * (0.03 + 0.04 * g) * (1.0 + 0.02 * groups)
                    if best is None or cost < best[0] - 1e-9:
                        best = (cost, per, head_split, 0)
                    if 1 < n + (1 if s.window > 0 else 0) <= 4:
                        rounds = (groups + sms - 1) // sms
                        fixed = 5.5 + 0.1 * g                                # start, and a warp merges a head at a time
                        cost = max(rounds * (fixed + per * wide * stage_us),
                                   fixed + max(once_us, again_us) / 1.05 + 1.0 * (rounds - 1))
                        if best_blk is None or cost < best_blk[0] - 1e-9:
                            best_blk = (cost, per, head_split, 1)
                    elif 4 < n + (1 if s.window > 0 else 0) <= 8:
                        rounds = (groups + sms // 2 - 1) // (sms // 2)       # clusters of two, a block an SM
                        fixed = 7.0 + 0.1 * g
                        cost = max(rounds * (fixed + per * wide * stage_us),
                                   fixed + max(once_us, again_us) / 1.05 + 3.0 * (rounds - 1))
                        if best_blk is None or cost < best_blk[0] - 1e-9:
                            best_blk = (cost, per, head_split, 2)
                if per >= pages_seq or per * wide >= 64:
                    break
                per *= 2
        if best_blk is not None and best_blk[0] < 0.95 * best[0]:
            best = best_blk
        return page * best[1], best[2], best[3]

    def _decode_twins(self, head_split: int, in_block: int):
        """``(head_split, twins)``: where a block (or a cluster) per item would take a group of 10 to 16 query heads
        as two blocks of instruction columns in one warp, the group is cut in two and the halves go to two warps
        that walk the same pages out of the same ring (``twins`` 2): the same work on twice the warps, whose chains
        of dependent matrix instructions then overlap a little.  64 sequences of 2,048 tokens with 32 query heads
        on 2 kv heads of 128: 32.0 against 33.4 us, of 4,096 tokens 50.6 against 52.5, of 512 tokens 15.8 against
        16.8."""
        g = self.spec.heads // self.spec.kv_heads // head_split
        if in_block and g > 8 and g % 2 == 0:
            return 2 * head_split, 2
        return head_split, 1

    def _chunks(self, max_kv_len: int, split: int) -> int:
        """The most chunks of ``split`` keys that a token's keys can touch."""
        n = (max_kv_len + split - 1) // split
        if self.spec.window > 0:
            n = min(n, (self.spec.window + split - 2) // split + 1)
        return max(1, n)

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.o.weight_bytes()


register_mixer("attention", Attention)
