// Attention of decoded tokens over the paged key/value cache: TMA into shared
// memory, both products on the tensor cores (mma.sync), bfloat16, heads of 64
// or 128, pages of 64 keys.
//
//   s[j] = (q . K[j]) * scale,  j in [max(0, pos - window + 1), pos]
//   out  = sum_j softmax(s)[j] * V[j]
//
// as in the reference's call of scaled-dot-product attention with an additive
// causal mask (src/model.cpp:539-548, 576-578); query head h reads key/value
// head h / (heads / kv_heads).
//
// A decoded token reads every key and value of its sequence once and does two
// multiply-adds per element: the kernel is bound by memory, and on the CUDA
// cores by the instructions that unpack and multiply the elements.  Here a
// page of keys is the 16-row operand of the matrix instruction (keys x
// features), the queries of the kv head's group are the 8 columns (two
// instructions side by side for groups of 9 to 16 query heads), and the
// scores come out transposed: S^T = K Q^T, then O^T = V^T P^T with V read
// through ldmatrix.trans and P^T made from the score registers by movmatrix.
// One page costs a warp 32 matrix instructions instead of some 600 scalar ones.
//
// Work item: (token, kv head, chunk of split_keys keys), one warp each.  A
// chunk is aligned to absolute positions, so for a given split_keys the way
// keys are grouped, and therefore every rounding, depends only on the token's
// own position: not on the batch, not on how the tokens were cut into steps.
// The chunks that hold keys are counted at the start (a token's position gives
// its chunks; shared memory holds the running sums), and the list of all of
// them, ordered by token, kv head and chunk, is cut into equal shares for the
// warps of a grid that fills the GPU once: sequences of unequal lengths are
// balanced, and a warp's chunks are neighbours, so that their pages follow one
// another in the block table.  Every warp has a ring of page buffers of its own,
// filled by TMA (128-byte swizzle, so that ldmatrix meets no bank conflicts)
// several pages ahead and across the ends of chunks; warps never wait for each
// other.  The chunks of a (token, kv head) are merged in chunk order by the
// warp that reports them last (a counter at the start of the scratch memory
// tells it); the scratch must be zero when it is first used and is left with
// zero counters by every launch.
//
// Scores, running maximum, running sum and the output accumulator are float32;
// the probabilities are rounded to bfloat16 for the second product.
//
// Two jobs of the step before attention can be done here (write_new, rotate):
// the half-split rotary encoding of the queries and of the token's own key
// (src/model.cpp:566-567), and that key's and value's way into the cache
// (src/model.cpp:569-574).  The warp that holds a token's last chunk takes its
// key and value from the projection's output, rotates the key, adds the pair to
// the softmax as one more key and writes it to the cache; the pages it reads
// then hold earlier steps' tokens only, so the page stream may start before
// the projection has finished (programmatic dependent launch).  This is for
// steps in which every sequence brings one token.
//
// Cache layout: pool[page][kv_head][slot][head_dim], page = block_table[row][pos / page_size].
#include "api.h"
#include "common.cuh"

#include <cuda.h>
#include <algorithm>
#include <math.h>
#include <type_traits>

namespace exl3 {

constexpr int AD_WARPS = 4;                                // warps that compute; each has a warp that copies for it
constexpr int AD_MAX_TWINS = 2;                            // computing warps that share a ring (see TW below)
constexpr int AD_PAGE = 64;
constexpr int AD_MAX_GROUP = 16;                           // query heads per kv head: one or two blocks of 8 instruction columns
// A stage holds the keys, then the values, of one page of one kv head (heads of 64) or of half a page (heads of
// 128): 8 KB each either way.
constexpr int AD_TILE_BYTES = 8192;
constexpr int AD_STAGE_BYTES = 2 * AD_TILE_BYTES;
constexpr int AD_STAGES = 3;
constexpr uint32_t AD_SMEM = AD_WARPS * AD_STAGES * AD_STAGE_BYTES + 1024;
constexpr int AD_MAX_TOKENS = 1024;                        // positions, sequences and chunk counts kept in shared memory
constexpr int AD_MAX_SPLITS = 256;                         // chunks of one (token, kv head)
constexpr int AD_COUNTER_SLOTS = 65536;                    // ints at the start of scratch, as in attention_simt.cu
constexpr uint32_t AD_WAIT_LIMIT = 1u << 24;               // polls of a few tens of cycles: a fraction of a second

static __device__ int g_ad_error = 0;

__device__ inline uint32_t ad_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ inline void ad_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ad_smem_u32(bar)), "r"(count));
}
__device__ inline void ad_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ad_smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded: false when the copy did not land within the limit.
__device__ inline bool ad_mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = ad_smem_u32(bar);
  for (uint32_t i = 0; i < AD_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
// The same for a warp that has nothing else to do: it sleeps between looks, so that it takes no issue slots
// from the warps that compute.
__device__ inline bool ad_mbar_wait_idle(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = ad_smem_u32(bar);
  for (uint32_t i = 0; i < AD_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
    __nanosleep(40);
  }
  return false;
}
__device__ inline void ad_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ad_smem_u32(bar)) : "memory");
}
// Thread-block clusters: a block's rank, a barrier over all threads of the cluster's blocks (release / acquire), and
// a float read from the same place in another block's shared memory.
__device__ inline uint32_t ad_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ inline void ad_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ inline float ad_ld_peer(const float* mine, uint32_t rank) {
  uint32_t addr;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(ad_smem_u32(mine)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ inline void ad_tma_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(ad_smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ inline void ad_ldsm(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ inline void ad_ldsm_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ inline void ad_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// An 8x8 matrix of 16-bit elements, one row of pairs per group of four lanes, transposed across the warp.
__device__ inline uint32_t ad_transpose(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ inline float ad_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ inline uint32_t ad_pack(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Record layout in scratch: [head_dim] accumulator, then max (base-2 units), then sum; as in attention_simt.cu.
//
// Under load every round trip to memory takes microseconds (the queues are full of pages on
// their way), so a warp waits for none of them per chunk: positions and sequences of all tokens
// are copied to shared memory at the start; page numbers are asked for 32 pages at a time, one
// batch ahead; queries are asked for one (token, kv head) ahead; records are stored and left
// behind, and one fence at the end of the warp's work covers them all before it draws tickets.
// NC: blocks of 8 query heads of a kv head's group (the columns of an instruction): 1 for groups of up to 8, 2 for
// up to 16.  Both blocks use the same key and value fragments, so a page is read from shared memory once.
// TW: computing warps of a ring.  With TW = 2 (in_block forms, NC = 1, kv_rep even) a block takes two groups of query
// heads of the same kv head: warp w and warp AD_WARPS + w walk the same chunk out of the same ring of pages, each
// with its own group's queries, so that a page comes into shared memory once for both and a scheduler has two
// warps to issue from.  A stage is free when both have read it (the barrier counts TW arrivals).
template <int HD, int NC, int TW>
__global__ void __launch_bounds__((TW + 1) * AD_WARPS * 32, 1)
attn_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const __nv_bfloat16* __restrict__ q, int64_t q_row_stride, __nv_bfloat16* __restrict__ out,
                   const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_pos,
                   const int* __restrict__ tok_seq, int T, int nh, int nkv, int window, float scale_log2,
                   int split_keys, int max_splits, float* __restrict__ scratch, int* __restrict__ counters,
                   const float* __restrict__ inv_freq, const float* __restrict__ inv_freq_lo, float pos_scale,
                   int rotate, int write_new,
                   __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, int kv_rep, int in_block) {
  // nkv counts groups of query heads that are worked on together.  With kv_rep = 2 the query heads of a kv head
  // are two such groups (g and g + 1 read kv head g / 2): twice the work items and two merges of half the size,
  // for steps with few tokens, where a single warp's merge of a wide group is what takes the time.
  constexpr int KS = HD == 64 ? 64 : 32;                 // keys of a stage
  constexpr int SPP = AD_PAGE / KS;                      // stages of a page
  constexpr int MT = KS / 16;                            // 16-key tiles of a stage
  constexpr int NJ = HD / 16;                            // 16-feature pieces of a head
  constexpr int NBOX = HD / 64;                          // 64-feature boxes (128-byte lines) of a row
  constexpr int BOX_BYTES = KS * 128;
  static_assert(KS * HD * 2 == AD_TILE_BYTES, "a stage is 8 KB of keys and 8 KB of values");
  extern __shared__ unsigned char ad_smem_raw[];
  __shared__ uint64_t full[AD_WARPS][AD_STAGES];         // a stage's copies have landed
  __shared__ uint64_t empty[AD_WARPS][AD_STAGES];        // the computing warp has read the stage
  __shared__ volatile unsigned s_asked[AD_WARPS];        // stages a ring's copier has asked for so far
  __shared__ int s_pos[AD_MAX_TOKENS], s_seq[AD_MAX_TOKENS];
  __shared__ int s_cum[AD_MAX_TOKENS + 1];               // chunks of the tokens before this one (per kv head)
  __shared__ float s_w[AD_WARPS][AD_MAX_SPLITS], s_l[AD_WARPS][AD_MAX_SPLITS];   // a merge's weights and sums
  __shared__ __align__(16) float2 s_rot[TW * AD_WARPS][64];   // a token's rotary angles (cos, sin), one table per computing warp
  // Warps 0 .. TW * AD_WARPS - 1 compute (warp w and, with TW = 2, warp AD_WARPS + w on ring w); the last AD_WARPS
  // warps ask for the copies into the rings (asked for by the computing warp itself, between two stages, they took
  // 200 to 400 of a stage's 1,100 to 1,300 cycles).
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp = wid % AD_WARPS;                       // the ring
  const bool copier = wid >= TW * AD_WARPS;
  const int tw = copier ? 0 : wid / AD_WARPS;            // which of the ring's computing warps
  const int gl = lane >> 2, tl = lane & 3;
  const int kv_heads = nkv / kv_rep;                     // key/value heads in the cache
  const uint32_t ring = ((ad_smem_u32(ad_smem_raw) + 1023u) & ~1023u) + warp * (AD_STAGES * AD_STAGE_BYTES);
  uint64_t* bars = full[warp];
  uint64_t* gone = empty[warp];
  if (lane == 0 && wid < AD_WARPS) {
    for (int s = 0; s < AD_STAGES; ++s) { ad_mbar_init(bars + s, 1); ad_mbar_init(gone + s, TW); }
    s_asked[warp] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  pdl_trigger();
  // Positions, sequences and page numbers are the step's inputs: no kernel of the step writes them.  When the
  // token's own key and value come from the projection (write_new), the cache pages this kernel reads hold
  // earlier steps' tokens only, so everything up to the first read of the queries, the first pages' copies
  // included, may run while the projection before this kernel is still at work.  Otherwise the position step
  // before this kernel has just written the newest page.
  if (!write_new) pdl_wait();

  // ---- every token's chunks, counted and summed ------------------------------------------------
  // A token at position pos reads keys lo .. pos; its chunks are the aligned pieces of split_keys
  // keys that this range touches, numbered from 0.
  auto first_key = [&](int pos) { return (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0; };
  for (int i = threadIdx.x; i < T; i += blockDim.x) {
    const int pos = __ldcg(tok_pos + i);
    s_pos[i] = pos;
    s_seq[i] = __ldcg(tok_seq + i);
    s_cum[i + 1] = min(pos / split_keys - first_key(pos) / split_keys + 1, max_splits);
  }
  if (threadIdx.x == 0) s_cum[0] = 0;
  __syncthreads();
  if (wid == 0) {
    const int per = (T + 31) / 32;                       // each lane sums a stretch of tokens, then the stretches are chained
    const int a = min(lane * per, T), b = min(a + per, T);
    int sum = 0;
    for (int i = a; i < b; ++i) sum += s_cum[i + 1];
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - sum;
    for (int i = a; i < b; ++i) { run += s_cum[i + 1]; s_cum[i + 1] = run; }
  }
  __syncthreads();

  const int G = nh / nkv;
  const int rec = HD + 2;
  auto chunks_of = [&](int t) { return s_cum[t + 1] - s_cum[t]; };
  auto base_of = [&](int t, int g) { return nkv * s_cum[t] + g * chunks_of(t); };   // index of chunk 0 of (t, g)
  // This warp's share: chunks i0 .. i1 - 1 of the list ordered by token, kv head, chunk: an equal contiguous share
  // of all of them, or (in_block: a block per (token, group of heads), at most AD_WARPS chunks each) the block's
  // item's chunk number `warp`, so that the item's chunks meet in this block's shared memory and no record of
  // them goes through global memory.
  const int n_chunks = nkv * s_cum[T];
  const int n_warps = gridDim.x * AD_WARPS, gw = blockIdx.x * AD_WARPS + warp;
  int i0 = (int)((int64_t)gw * n_chunks / n_warps), i1 = (int)((int64_t)(gw + 1) * n_chunks / n_warps);
  // in_block = 2: the item belongs to a cluster of two blocks, whose eight computing warps take its up to eight
  // chunks; the first block merges, reading the second one's records out of its shared memory.
  const int pair = in_block == 2 ? 2 : 1;
  const uint32_t crank = pair == 2 ? ad_cluster_rank() : 0u;
  const int item = in_block ? (int)blockIdx.x / pair : 0;
  const int t_blk = item / (nkv / TW), g_blk = item % (nkv / TW) * TW + tw;   // a ring's copier: as its first computing warp
  if (in_block) {
    const int mine = (int)crank * AD_WARPS + warp;       // this warp's chunk of the item
    i0 = base_of(t_blk, g_blk) + mine;
    i1 = mine < chunks_of(t_blk) ? i0 + 1 : i0;
  }
  // in_block: chunk sp's record lies at the start of warp sp's ring of pages, which that warp no longer needs
  // when it has walked its chunk
  float* const rec_blk = reinterpret_cast<float*>(ad_smem_raw + ((1024u - (ad_smem_u32(ad_smem_raw) & 1023u)) & 1023u));
  constexpr int REC_BLK_STRIDE = AD_STAGES * AD_STAGE_BYTES / 4;      // floats from one warp's ring to the next
  // the token whose chunks hold index i
  auto token_of = [&](int i) {
    int lo = 0, hi = T - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (nkv * s_cum[mid] <= i) lo = mid; else hi = mid - 1;
    }
    return lo;
  };
  // keys of chunk sp of token t
  auto chunk_keys = [&](int t, int sp, int& c_lo, int& c_hi) {
    const int pos = s_pos[t], lo = first_key(pos);
    const int c = lo / split_keys + sp;
    c_lo = max(lo, c * split_keys);
    c_hi = min(write_new ? pos : pos + 1, (c + 1) * split_keys);   // the new token's key is not in the cache yet
  };

  // ldmatrix addresses inside a swizzled tile: row r at r * 128 bytes, its 16-byte piece c at c ^ (r & 7)
  const uint32_t k_row = ((lane & 7) + ((lane >> 3) & 1) * 8) * 128;
  const uint32_t v_row = ((lane & 7) + ((lane >> 4) & 1) * 8) * 128 + AD_TILE_BYTES;   // values follow the keys
  uint32_t k_col[4], v_col[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    k_col[j] = (uint32_t)(((2 * j + (lane >> 4)) ^ (lane & 7)) << 4);
    v_col[j] = (uint32_t)(((2 * j + ((lane >> 3) & 1)) ^ (lane & 7)) << 4);
  }

  // ---- the producer: pages in the order the chunks will want them -----------------------------
  // The chunks of one (token, kv head) that this warp holds are neighbours, and so are their
  // pages: a run.  Page numbers come 32 at a time (lane i holds page0 + i), one batch ahead.  The unit
  // of copying is a stage's worth of keys (KS: a page, or half of one).
  struct Batch { int t, g, gk, page0, sub_a, sub_b; bool some; };   // stages sub_a .. sub_b of the run are still ahead; gk: the kv head of group g
  auto run_of = [&](int t, int g, Batch& bt) {           // the pages of (t, g) inside i0 .. i1
    const int base = base_of(t, g);
    const int sp_a = max(i0 - base, 0), sp_b = min(i1 - base, chunks_of(t)) - 1;
    int c_lo, c_hi;
    chunk_keys(t, sp_a, c_lo, c_hi);
    bt.sub_a = c_lo / KS;
    bt.page0 = bt.sub_a / SPP;
    chunk_keys(t, sp_b, c_lo, c_hi);
    bt.sub_b = (c_hi + KS - 1) / KS - 1;                 // below sub_a when the run holds no cached key
    bt.t = t;
    bt.g = g;
    bt.gk = g / kv_rep;
    bt.some = true;
  };
  auto batch_after = [&](const Batch& cur, Batch& nx) {
    nx = cur;
    if ((cur.page0 + 32) * SPP <= cur.sub_b) { nx.page0 = cur.page0 + 32; nx.sub_a = nx.page0 * SPP; return; }
    int t = cur.t, g = cur.g + 1;
    if (g == nkv) { g = 0; ++t; }
    if (t >= T || base_of(t, g) >= i1) { nx.some = false; return; }
    run_of(t, g, nx);
  };
  auto fetch = [&](const Batch& bt) {
    const int idx = bt.page0 + lane;
    return (bt.some && bt.sub_a <= bt.sub_b && idx <= bt.sub_b / SPP)
               ? __ldcg(block_table + (int64_t)s_seq[bt.t] * bt_stride + idx) : 0;
  };
  Batch cur_b, nxt_b;
  cur_b.some = false;
  int cur_pages = 0, nxt_pages = 0, p_pi = 1, p_end = 0;   // stages p_pi .. p_end of the current batch are still to ask for
  int t0 = 0, g0 = 0, sp0 = 0;
  nxt_b.some = false;
  if (i0 < i1) {
    t0 = token_of(i0);
    const int r = i0 - nkv * s_cum[t0];
    g0 = r / chunks_of(t0);
    sp0 = r - g0 * chunks_of(t0);
    run_of(t0, g0, nxt_b);
  }
  nxt_pages = fetch(nxt_b);
  uint32_t pn = 0;                                       // pages asked for
  auto produce = [&]() -> bool {
    while (p_pi > p_end) {
      if (!nxt_b.some) return false;                     // no page left for this ring
      cur_b = nxt_b;
      cur_pages = nxt_pages;
      p_pi = cur_b.sub_a;
      p_end = min((cur_b.page0 + 32) * SPP - 1, cur_b.sub_b);
      batch_after(cur_b, nxt_b);
      nxt_pages = fetch(nxt_b);
    }
    const int pg = __shfl_sync(0xffffffffu, cur_pages, p_pi / SPP - cur_b.page0);
    if (lane == 0) {
      const uint32_t s = pn % AD_STAGES;
      const uint32_t dst = ring + s * AD_STAGE_BYTES;
      const int row = (pg * kv_heads + cur_b.gk) * AD_PAGE + (p_pi % SPP) * KS;   // no division here: this runs once a stage
      ad_mbar_expect_tx(bars + s, AD_STAGE_BYTES);
#pragma unroll
      for (int b = 0; b < NBOX; ++b) {
        ad_tma_2d(dst + b * BOX_BYTES, &map_k, bars + s, 64 * b, row);
        ad_tma_2d(dst + AD_TILE_BYTES + b * BOX_BYTES, &map_v, bars + s, 64 * b, row);
      }
    }
    ++p_pi;
    ++pn;
    if (lane == 0) s_asked[warp] = pn;
    return true;
  };
  if (copier) {
    // ---- a ring's copies: a stage as soon as the computing warp is done with what was in it ----
    bool fine = true;
    for (;;) {
      if (pn >= AD_STAGES && !ad_mbar_wait_idle(gone + pn % AD_STAGES, ((pn / AD_STAGES) - 1) & 1)) { fine = false; break; }
      if (!produce()) break;
    }
    if (!fine) {
      // the computing warp never came: say so, and give the copies in flight a bounded time to land
      if (lane == 0) atomicExch(&g_ad_error, 1);
      for (uint32_t u = pn > (uint32_t)AD_STAGES ? pn - AD_STAGES : 0; u < pn; ++u)
        if (!ad_mbar_wait(bars + u % AD_STAGES, (u / AD_STAGES) & 1)) break;
    }
  }

  // Q^T as the right operand: column gl of block c is query head 8 c + gl of the group, zero beyond the group
  auto load_q = [&](int t, int g, bool some, uint32_t (&qq)[NC][NJ][2]) {
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const unsigned* qrow = reinterpret_cast<const unsigned*>(q + (int64_t)t * q_row_stride +
                                                               (int64_t)(g * G + 8 * c + gl) * HD);
      const bool live = some && 8 * c + gl < G;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        qq[c][j][0] = live ? __ldcg(qrow + 8 * j + tl) : 0u;
        qq[c][j][1] = live ? __ldcg(qrow + 8 * j + tl + 4) : 0u;
      }
    }
  };
  // the (token, kv head) after (t, g), if this warp holds chunks of it
  auto next_run = [&](int t, int g, int& nt, int& ng) {
    nt = t;
    ng = g + 1;
    if (ng == nkv) { ng = 0; ++nt; }
    return nt < T && base_of(nt, ng) < i1;
  };

  // ---- the position encoding, when it is this kernel's to apply -------------------------------
  // Half-split rotary pairs (d, d + HD / 2) with angle pos * pos_scale * (inv_freq[d] + inv_freq_lo[d]), as rope_kv_write does it
  // (elementwise.cu).  A thread's fragment holds features 16 j + 2 tl + 8 h + e: a pair's two halves are its
  // pieces j and j + NJ / 2.
  // A token's HD / 2 angles are computed once, two or so per lane, and kept in the warp's table (cos, sin):
  // the token's query heads of every kv head and its own key all turn by them.
  float2* rot_tab = s_rot[copier ? 0 : wid];
  int rot_t = -1;                                        // the token whose angles the table holds
  auto angles_of = [&](int t) {
    if (t == rot_t) return;
    __syncwarp();                                        // the table's last readers are done
    const float p = (float)s_pos[t] * pos_scale;
    for (int d = lane; d < HD / 2; d += 32) {
      float sn, cs;
      rope_sincos(p, __ldg(inv_freq + d), inv_freq_lo ? __ldg(inv_freq_lo + d) : 0.0f, &sn, &cs);
      rot_tab[d] = make_float2(cs, sn);
    }
    __syncwarp();
    rot_t = t;
  };
  auto rotate_at = [&](int t, uint32_t (&f)[NJ][2]) {
    angles_of(t);
#pragma unroll
    for (int j = 0; j < NJ / 2; ++j) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float4 a = *reinterpret_cast<const float4*>(rot_tab + 16 * j + 2 * tl + 8 * h);   // pairs d, d + 1
        const uint32_t x0 = f[j][h], x1 = f[j + NJ / 2][h];
        const float a0 = __uint_as_float(x0 << 16), a1 = __uint_as_float(x1 << 16);
        const float b0 = __uint_as_float(x0 & 0xffff0000u), b1 = __uint_as_float(x1 & 0xffff0000u);
        const float r0a = a0 * a.x - a1 * a.y, r1a = a1 * a.x + a0 * a.y;
        const float r0b = b0 * a.z - b1 * a.w, r1b = b1 * a.z + b0 * a.w;
        f[j][h] = ad_pack(r0a, r0b);
        f[j + NJ / 2][h] = ad_pack(r1a, r1b);
      }
    }
  };

  // ---- merging the chunks of a (token, kv head): the same sums in chunk order, whoever does it --
  // HG query heads of the group side by side, 32 / HG lanes each: the warp waits for memory once for all the
  // chunks' maxima and sums together with the first MB chunks of accumulators, and once per MB chunks after
  // them, however many heads the group has.
  auto merge_heads = [&](auto hg_c, int mt, int mg, int n0) {
    constexpr int HG = decltype(hg_c)::value;
    constexpr int LPH = 32 / HG;                         // lanes of a head
    constexpr int DPL = HD / LPH;                        // features of a lane: the pairs i * LPH + lih of the head
    constexpr int F2 = DPL / 2;
    constexpr int MB = DPL <= 4 ? 16 : 64 / DPL;         // chunks asked for at once
    float* wv = s_w[warp];
    float* lv = s_l[warp];
    const int n_rec = chunks_of(mt);
    const int heads = min(HG, G - n0);
    const float* base = scratch + ((int64_t)mt * nh + mg * G + n0) * max_splits * rec;   // a head's records: max_splits of them
    const int n_pairs = heads * n_rec;
    const int nn = lane / LPH, lih = lane % LPH;
    const float* hb = base + (int64_t)nn * max_splits * rec;
    float2 v[MB][F2];
    auto ask = [&](int s0) {                             // the accumulators of chunks s0 .. s0 + MB - 1
#pragma unroll
      for (int u = 0; u < MB; ++u) {
        const float2* r = reinterpret_cast<const float2*>(hb + (int64_t)(s0 + u) * rec);
        const bool in = nn < heads && s0 + u < n_rec;
#pragma unroll
        for (int i = 0; i < F2; ++i) v[u][i] = in ? __ldcg(r + i * LPH + lih) : make_float2(0.0f, 0.0f);
      }
    };
    for (int p = lane; p < n_pairs; p += 32) {
      const int n = p / n_rec, s2 = p - n * n_rec;
      const float* r = base + ((int64_t)n * max_splits + s2) * rec + HD;
      wv[p] = __ldcg(r);
      lv[p] = __ldcg(r + 1);
    }
    ask(0);                                              // on their way while the weights are worked out
    __syncwarp();
    float my_ll = 1.0f;
#pragma unroll
    for (int n = 0; n < HG; ++n) {
      if (n < heads) {
        float M = -INFINITY;
        for (int s2 = lane; s2 < n_rec; s2 += 32) M = fmaxf(M, wv[n * n_rec + s2]);
        M = warp_max(M);
        float ll = 0.0f;
        for (int s2 = lane; s2 < n_rec; s2 += 32) {
          const float w = ad_exp2(wv[n * n_rec + s2] - M);
          wv[n * n_rec + s2] = w;
          ll += lv[n * n_rec + s2] * w;
        }
        ll = warp_sum(ll);
        if (nn == n) my_ll = ll;
      }
    }
    __syncwarp();
    if (nn < heads) {
      const float* wn = wv + nn * n_rec;
      float acc[DPL];
#pragma unroll
      for (int e = 0; e < DPL; ++e) acc[e] = 0.0f;
      for (int s0 = 0; s0 < n_rec; s0 += MB) {
        if (s0 > 0) ask(s0);
#pragma unroll
        for (int u = 0; u < MB; ++u) {
          const float w = s0 + u < n_rec ? wn[s0 + u] : 0.0f;
#pragma unroll
          for (int i = 0; i < F2; ++i) {
            acc[2 * i] += v[u][i].x * w;
            acc[2 * i + 1] += v[u][i].y * w;
          }
        }
      }
      __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(out + ((int64_t)mt * nh + mg * G + n0 + nn) * HD);
#pragma unroll
      for (int i = 0; i < F2; ++i)
        dst[i * LPH + lih] = __floats2bfloat162_rn(acc[2 * i] / my_ll, acc[2 * i + 1] / my_ll);
    }
    __syncwarp();                                        // before the next heads' weights
  };
  auto merge = [&](int mt, int mg) {
    const int n_rec = chunks_of(mt);
    int hg = 1;                                          // as many heads at once as the weights' table takes
    while (hg < G && hg < 8 && 2 * hg * n_rec <= AD_MAX_SPLITS) hg *= 2;
    for (int n0 = 0; n0 < G; n0 += hg) {
      switch (hg) {
        case 1: merge_heads(std::integral_constant<int, 1>{}, mt, mg, n0); break;
        case 2: merge_heads(std::integral_constant<int, 2>{}, mt, mg, n0); break;
        case 4: merge_heads(std::integral_constant<int, 4>{}, mt, mg, n0); break;
        default: merge_heads(std::integral_constant<int, 8>{}, mt, mg, n0); break;
      }
    }
    if (lane == 0) counters[(int64_t)mt * nkv + mg] = 0;   // zero again for the next launch
  };

  // ---- the consumer: chunk after chunk ---------------------------------------------------------
  uint32_t cn = 0;                                       // pages used
  bool ok = true;
  int t = t0, g = g0, sp = sp0;
  uint32_t qb[NC][NJ][2], qn[NC][NJ][2];
  int nt = 0, ng = 0;
  bool nsome = false;
  if (!copier) {
  if (rotate && i0 < i1) angles_of(t0);                  // positions are the step's inputs
  if (write_new) pdl_wait();                             // from here on the projection's output is read
  if (i0 < i1) {
    load_q(t, g, true, qb);
    nsome = next_run(t, g, nt, ng);
    load_q(nt, ng, nsome, qn);                           // used when this warp gets to (nt, ng)
    if (rotate) {
#pragma unroll
      for (int c = 0; c < NC; ++c) rotate_at(t, qb[c]);
    }
  }
#pragma unroll 1
  for (int i = i0; i < i1 && ok; ++i) {
    int c_lo, c_hi;
    chunk_keys(t, sp, c_lo, c_hi);
    const int first_sub = c_lo / KS, last_sub = c_lo < c_hi ? (c_hi - 1) / KS : first_sub - 1;
    // The token's own key and value: the warp with the token's last chunk takes them from the projection's
    // output (asked for now, used after the chunk's pages), rotates the key, adds the pair to the softmax as
    // one more key and writes it to the cache.
    const bool has_new = write_new && sp == chunks_of(t) - 1;
    uint32_t kf[NJ][2];
    unsigned short vf[2 * NJ];
    int new_page = 0;
    if (has_new) {
      const __nv_bfloat16* row = q + (int64_t)t * q_row_stride;
      const unsigned* krow = reinterpret_cast<const unsigned*>(row + (int64_t)(nh + g / kv_rep) * HD);
      const unsigned short* vrow = reinterpret_cast<const unsigned short*>(row + (int64_t)(nh + nkv / kv_rep + g / kv_rep) * HD);
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        kf[j][0] = __ldcg(krow + 8 * j + tl);
        kf[j][1] = __ldcg(krow + 8 * j + tl + 4);
        vf[2 * j] = __ldcg(vrow + 16 * j + gl);
        vf[2 * j + 1] = __ldcg(vrow + 16 * j + gl + 8);
      }
      new_page = __ldcg(block_table + (int64_t)s_seq[t] * bt_stride + s_pos[t] / AD_PAGE);
    }
    float m[NC][2], l[NC][2];
    float o[NC][NJ][4];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      m[c][0] = m[c][1] = -INFINITY;
      l[c][0] = l[c][1] = 0.0f;
#pragma unroll
      for (int a = 0; a < NJ; ++a) {
#pragma unroll
        for (int e = 0; e < 4; ++e) o[c][a][e] = 0.0f;
      }
    }
#pragma unroll 1
    for (int pi = first_sub; pi <= last_sub; ++pi) {
      const uint32_t st = cn % AD_STAGES;
      if (!ad_mbar_wait(bars + st, (cn / AD_STAGES) & 1)) { ok = false; break; }
      const uint32_t kb = ring + st * AD_STAGE_BYTES;
      // S^T = K Q^T: s[c][a] holds keys 16 a + gl (elements 0, 1) and + 8 (2, 3) for queries 2 tl, 2 tl + 1 of block c
      float s[NC][MT][4];
#pragma unroll
      for (int a = 0; a < MT; ++a) {
        float s_hi[NC][4];                                 // features 64 .. of a head of 128: a chain of its own
#pragma unroll
        for (int c = 0; c < NC; ++c) {
#pragma unroll
          for (int e = 0; e < 4; ++e) { s[c][a][e] = 0.0f; s_hi[c][e] = 0.0f; }
        }
#pragma unroll
        for (int j = 0; j < NJ; ++j) {                     // features 16 j ..: box j / 4, its piece j % 4
          uint32_t f[4];
          ad_ldsm(f, kb + (j >> 2) * BOX_BYTES + a * 2048 + k_row + k_col[j & 3]);
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            if (j < 4) ad_mma(s[c][a], f, qb[c][j][0], qb[c][j][1]);
            else ad_mma(s_hi[c], f, qb[c][j][0], qb[c][j][1]);
          }
        }
        if (NJ > 4) {
#pragma unroll
          for (int c = 0; c < NC; ++c) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[c][a][e] += s_hi[c][e];
          }
        }
      }
      const int key0 = pi * KS;
      if (key0 < c_lo || key0 + KS > c_hi) {
#pragma unroll
        for (int a = 0; a < MT; ++a) {
          const int ka = key0 + 16 * a + gl, kb2 = ka + 8;
          const bool da = (ka < c_lo) | (ka >= c_hi), db = (kb2 < c_lo) | (kb2 >= c_hi);
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            s[c][a][0] = da ? -INFINITY : s[c][a][0];
            s[c][a][1] = da ? -INFINITY : s[c][a][1];
            s[c][a][2] = db ? -INFINITY : s[c][a][2];
            s[c][a][3] = db ? -INFINITY : s[c][a][3];
          }
        }
      }
      // P^T as the right operand of the second product, by transposing 8x8 pieces across the warp
      uint32_t pb[NC][MT][2];
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        float mx[2], corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mx[h] = fmaxf(s[c][0][h], s[c][0][h + 2]);
#pragma unroll
          for (int a = 1; a < MT; ++a) mx[h] = fmaxf(mx[h], fmaxf(s[c][a][h], s[c][a][h + 2]));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
          const float mn = fmaxf(m[c][h], mx[h] * scale_log2);   // a page in the chunk has a live key: finite
          corr[h] = ad_exp2(m[c][h] - mn);                        // 0 on the first page
          m[c][h] = mn;
        }
#pragma unroll
        for (int a = 0; a < MT; ++a) {
          const float p0 = ad_exp2(fmaf(s[c][a][0], scale_log2, -m[c][0]));
          const float p1 = ad_exp2(fmaf(s[c][a][1], scale_log2, -m[c][1]));
          const float p2 = ad_exp2(fmaf(s[c][a][2], scale_log2, -m[c][0]));
          const float p3 = ad_exp2(fmaf(s[c][a][3], scale_log2, -m[c][1]));
          l[c][0] = l[c][0] * (a == 0 ? corr[0] : 1.0f) + (p0 + p2);
          l[c][1] = l[c][1] * (a == 0 ? corr[1] : 1.0f) + (p1 + p3);
          pb[c][a][0] = ad_transpose(ad_pack(p0, p1));
          pb[c][a][1] = ad_transpose(ad_pack(p2, p3));
        }
#pragma unroll
        for (int d = 0; d < NJ; ++d) {
          o[c][d][0] *= corr[0];
          o[c][d][1] *= corr[1];
          o[c][d][2] *= corr[0];
          o[c][d][3] *= corr[1];
        }
      }
      // O^T += V^T P^T: o[c][d] holds features 16 d + gl (elements 0, 1) and + 8 (2, 3) for queries 2 tl, 2 tl + 1
#pragma unroll
      for (int a = 0; a < MT; ++a) {
#pragma unroll
        for (int d = 0; d < NJ; ++d) {
          uint32_t f[4];
          ad_ldsm_t(f, kb + (d >> 2) * BOX_BYTES + a * 2048 + v_row + v_col[d & 3]);
#pragma unroll
          for (int c = 0; c < NC; ++c) ad_mma(o[c][d], f, pb[c][a][0], pb[c][a][1]);
        }
      }
      __syncwarp();                                      // every lane has read the stage
      if (lane == 0) ad_mbar_arrive(gone + st);          // its copier may ask for the stage AD_STAGES ahead
      ++cn;
    }
    // the ring's other computing warp may still read the stage where this one's record goes
    if (TW == 2) asm volatile("bar.sync %0, 64;" ::"r"(1 + warp) : "memory");
    if (!ok) break;
    if (has_new) {
      if (rotate) rotate_at(t, kf);
      // to the cache, for the steps to come: the key from the lanes of query column 0, the value as it is
      // (with kv_rep = 2 both groups of a kv head write the same key and value to the same place)
      const int64_t at = (((int64_t)new_page * (nkv / kv_rep) + g / kv_rep) * AD_PAGE + (s_pos[t] % AD_PAGE)) * HD;
      if (new_page >= 0) {
        if (gl == 0) {
          unsigned* kdst = reinterpret_cast<unsigned*>(k_pool + at);
#pragma unroll
          for (int j = 0; j < NJ; ++j) {
            kdst[8 * j + tl] = kf[j][0];
            kdst[8 * j + tl + 4] = kf[j][1];
          }
        }
        if (lane < HD / 8) {
          const uint4* vsrc = reinterpret_cast<const uint4*>(q + (int64_t)t * q_row_stride +
                                                             (int64_t)(nh + nkv / kv_rep + g / kv_rep) * HD);
          reinterpret_cast<uint4*>(v_pool + at)[lane] = __ldcg(vsrc + lane);
        }
      }
      // its score against this lane group's queries (column gl of each block), then to the lanes that hold those
      // columns' state
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            dot = fmaf(__uint_as_float(qb[c][j][h] << 16), __uint_as_float(kf[j][h] << 16), dot);
            dot = fmaf(__uint_as_float(qb[c][j][h] & 0xffff0000u), __uint_as_float(kf[j][h] & 0xffff0000u), dot);
          }
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float sc = __shfl_sync(0xffffffffu, dot, (2 * tl + h) * 4) * scale_log2;
          const float mn = fmaxf(m[c][h], sc);
          const float corr = ad_exp2(m[c][h] - mn);              // 0 when the cache held no key of this chunk
          const uint32_t pp = ad_pack(ad_exp2(sc - mn), 0.0f);   // rounded as the other probabilities are
          const float pr = __uint_as_float(pp << 16);
          m[c][h] = mn;
          l[c][h] = l[c][h] * corr + (gl == 0 ? pr : 0.0f);      // the sum over lane groups below counts it once
#pragma unroll
          for (int d = 0; d < NJ; ++d) {
            o[c][d][h] = o[c][d][h] * corr + pr * __uint_as_float((uint32_t)vf[2 * d] << 16);
            o[c][d][h + 2] = o[c][d][h + 2] * corr + pr * __uint_as_float((uint32_t)vf[2 * d + 1] << 16);
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < NC; ++c) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        l[c][h] += __shfl_xor_sync(0xffffffffu, l[c][h], 4);
        l[c][h] += __shfl_xor_sync(0xffffffffu, l[c][h], 8);
        l[c][h] += __shfl_xor_sync(0xffffffffu, l[c][h], 16);
      }
    }
    // ---- the chunk's result ------------------------------------------------------------------
    const int n_rec = chunks_of(t);
#pragma unroll
    for (int c = 0; c < NC; ++c) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int n = 8 * c + 2 * tl + h;
        if (n >= G) continue;
        const int head = g * G + n;
        if (n_rec == 1) {
          __nv_bfloat16* dst = out + ((int64_t)t * nh + head) * HD;
          const float inv = 1.0f / l[c][h];
#pragma unroll
          for (int d = 0; d < NJ; ++d) {
            dst[16 * d + gl] = __float2bfloat16(o[c][d][h] * inv);
            dst[16 * d + gl + 8] = __float2bfloat16(o[c][d][h + 2] * inv);
          }
        } else {
          float* sc = in_block ? rec_blk + (sp % AD_WARPS) * REC_BLK_STRIDE + (tw * G + n) * rec
                               : scratch + (((int64_t)t * nh + head) * max_splits + sp) * rec;
#pragma unroll
          for (int d = 0; d < NJ; ++d) {
            sc[16 * d + gl] = o[c][d][h];
            sc[16 * d + gl + 8] = o[c][d][h + 2];
          }
          if (gl == 0) { sc[HD] = m[c][h]; sc[HD + 1] = l[c][h]; }
        }
      }
    }
    // on to the next chunk; a new (token, kv head) brings its queries, asked for a run ago
    if (++sp == n_rec) {
      sp = 0;
      t = nt;
      g = ng;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) { qb[c][j][0] = qn[c][j][0]; qb[c][j][1] = qn[c][j][1]; }
        if (rotate && i + 1 < i1) rotate_at(t, qb[c]);
      }
      if (nsome) {
        nsome = next_run(t, g, nt, ng);
        load_q(nt, ng, nsome, qn);
      }
    }
  }
  }
  if (in_block) {
    if (!copier && !ok) {
      if (lane == 0) atomicExch(&g_ad_error, 1);
      for (; cn < s_asked[warp]; ++cn) {
        if (!ad_mbar_wait(bars + cn % AD_STAGES, (cn / AD_STAGES) & 1)) break;
      }
    }
    // every warp comes here, whatever its share and its outcome
    if (pair == 2) ad_cluster_sync(); else __syncthreads();
    const int n_rec = chunks_of(t_blk);
    if (n_rec > 1 && !copier && crank == 0) {
      // chunks 4 .. 7 lie in the cluster's other block (fetching them all in one trip before the merge, instead of
      // a remote read per use, changed nothing: 13.5 against 13.4 us)
      auto rec_at = [&](const float* hb, int s2, int d) {
        const float* p = hb + (s2 % AD_WARPS) * REC_BLK_STRIDE + d;
        return s2 < AD_WARPS ? *p : ad_ld_peer(p, 1);
      };
      // the item's chunks, in chunk order; a warp takes every fourth head, a lane HD / 32 features
      for (int n = warp; n < G; n += AD_WARPS) {
        const float* hb = rec_blk + (tw * G + n) * rec;
        float M = -INFINITY;
        for (int s2 = 0; s2 < n_rec; ++s2) M = fmaxf(M, rec_at(hb, s2, HD));
        float w[2 * AD_WARPS], ll = 0.0f;
#pragma unroll
        for (int s2 = 0; s2 < 2 * AD_WARPS; ++s2) {
          w[s2] = s2 < n_rec ? ad_exp2(rec_at(hb, s2, HD) - M) : 0.0f;
          ll += s2 < n_rec ? rec_at(hb, s2, HD + 1) * w[s2] : 0.0f;
        }
        __nv_bfloat16* dst = out + ((int64_t)t_blk * nh + g_blk * G + n) * HD;
#pragma unroll
        for (int e = 0; e < HD / 32; ++e) {
          const int d = e * 32 + lane;
          float acc = 0.0f;
#pragma unroll
          for (int s2 = 0; s2 < 2 * AD_WARPS; ++s2) acc += s2 < n_rec ? rec_at(hb, s2, d) * w[s2] : 0.0f;
          dst[d] = __float2bfloat16(acc / ll);
        }
      }
    }
    if (pair == 2) ad_cluster_sync();                    // the other block's records stay until they are read
  } else if (copier) {
    // nothing left to do: the ring's copies are asked for, and the computing warp waits for each of them
  } else if (ok) {
    // All of this warp's records are written.  One fence for all of them, then a ticket per chunk,
    // lanes side by side; the chunks of a (token, kv head) are merged by the warp that draws the
    // last ticket.  Which warp that is varies; what it computes does not.
    __threadfence();
    __syncwarp();
    for (int k0 = i0; k0 < i1; k0 += 32) {
      int mt = 0, mg = 0;
      bool last = false;
      if (k0 + lane < i1) {
        mt = token_of(k0 + lane);
        const int n_rec = chunks_of(mt);
        mg = (k0 + lane - nkv * s_cum[mt]) / n_rec;
        if (n_rec > 1) last = atomicAdd(counters + (int64_t)mt * nkv + mg, 1) == n_rec - 1;
      }
      unsigned todo = __ballot_sync(0xffffffffu, last);
      if (todo) __threadfence();
      while (todo) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        merge(__shfl_sync(0xffffffffu, mt, src), __shfl_sync(0xffffffffu, mg, src));
      }
    }
  } else {
    // A copy did not land in time: say so, and give the copies still in flight a bounded time to
    // land before the block's shared memory goes away.
    if (lane == 0) atomicExch(&g_ad_error, 1);
    for (; cn < s_asked[warp]; ++cn) {
      if (!ad_mbar_wait(bars + cn % AD_STAGES, (cn / AD_STAGES) & 1)) break;
    }
  }
}

// ---- host side --------------------------------------------------------------------------

typedef CUresult (*AdEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AdEncodeFn ad_encode_fn() {
  static AdEncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<AdEncodeFn>(p);
  }();
  return fn;
}
// [rows, hd] bfloat16, rows packed; boxes of 64 features x box_rows rows, 128B swizzle.
static int ad_make_map(CUtensorMap* map, const void* ptr, int64_t rows, int hd, int box_rows) {
  AdEncodeFn fn = ad_encode_fn();
  if (!fn) { set_error("attn_decode: the driver has no cuTensorMapEncodeTiled"); return ERR_UNSUPPORTED; }
  const cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("attn_decode: cuTensorMapEncodeTiled failed with %d", (int)r); return ERR_BAD_ARGUMENT; }
  return 0;
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_attn_decode_supported(int dtype, int T, int nh, int nkv, int hd, int page, int split_keys,
                                          int max_splits) {
  return dtype == DT_BF16 && (hd == 64 || hd == 128) && page == AD_PAGE && T >= 0 && T <= AD_MAX_TOKENS && nkv >= 1 &&
         nh % nkv == 0 && nh / nkv <= AD_MAX_GROUP && split_keys > 0 && split_keys % AD_PAGE == 0 &&
         max_splits >= 1 && max_splits <= AD_MAX_SPLITS && (max_splits == 1 || (int64_t)T * nkv <= AD_COUNTER_SLOTS);
}

extern "C" int exl3_attn_decode_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_ad_error, sizeof(int));
  if (v) { int z = 0; cudaMemcpyToSymbol(g_ad_error, &z, sizeof(int)); }
  return v;
}

// Same arguments and the same scratch layout as exl3_attn_tokens; n_pool_rows = pages * kv_heads * 64.
// With write_new, q is the fused q|k|v output of the projection and every token is its sequence's only new one:
// the kernel takes the token's key and value from there, adds them to its softmax and writes them to the cache
// (which holds the positions before it).  With rot = hd it also applies the half-split rotary encoding
// (angle pos * pos_scale * (inv_freq[d] + inv_freq_lo[d]), hd / 2 frequencies each, inv_freq_lo may be null) to the
// queries and the new key; rot = 0: none.
extern "C" int exl3_attn_decode(const void* q, int64_t q_row_stride, void* out, void* k_pool, void* v_pool,
                                int64_t n_pool_rows, const int* block_table, int bt_stride, const int* tok_pos,
                                const int* tok_seq, int T, int nh, int nkv, int hd, int page, int window,
                                float scale, int split_keys, int max_splits, float* scratch, size_t scratch_bytes,
                                const float* inv_freq, const float* inv_freq_lo, int rot, float pos_scale,
                                int write_new, int head_split, int in_block, int twins, cudaStream_t stream) {
  if (T == 0) return 0;
  if (in_block < 0 || in_block > 2 || (in_block && (max_splits < 1 || max_splits > in_block * AD_WARPS))) {
    set_error("attn_decode: in_block is 0, 1 (a block merges up to %d chunks of a (token, group of heads) itself) or 2 "
              "(a cluster of two blocks, up to %d); got %d with %d chunks", AD_WARPS, 2 * AD_WARPS, in_block, max_splits);
    return ERR_BAD_ARGUMENT;
  }
  if (head_split < 1 || head_split > AD_MAX_GROUP || nkv < 1 || nh % nkv != 0 || (nh / nkv) % head_split != 0) {
    set_error("attn_decode: head_split must divide the %d query heads of a kv head; got %d", nkv > 0 ? nh / nkv : 0, head_split);
    return ERR_BAD_ARGUMENT;
  }
  if (twins != 1 && (twins != AD_MAX_TWINS || !in_block || head_split % twins != 0 || nh / (nkv * head_split) > 8)) {
    set_error("attn_decode: twins is 1 or %d (two groups of up to 8 query heads of a kv head in one block: in_block 1 or 2 "
              "and an even head_split); got %d with in_block %d, head_split %d, %d heads a group", AD_MAX_TWINS, twins,
              in_block, head_split, nh / (nkv * head_split));
    return ERR_BAD_ARGUMENT;
  }
  if (nh < 1 || nkv < 1 || window < 0 || !(scale > 0.0f) ||
      !exl3_attn_decode_supported(DT_BF16, T, nh, nkv, hd, page, split_keys, max_splits)) {
    set_error("attn_decode: needs bfloat16, head_dim 64 or 128, pages of 64, at most %d tokens, %d query heads per kv "
              "head and %d chunks of whole pages; got T=%d heads=%d kv_heads=%d head_dim=%d page=%d window=%d "
              "split_keys=%d max_splits=%d", AD_MAX_TOKENS, AD_MAX_GROUP, AD_MAX_SPLITS, T, nh, nkv, hd, page,
              window, split_keys, max_splits);
    return ERR_UNSUPPORTED;
  }
  if ((rot != 0 && rot != hd) || (rot != 0 && inv_freq == nullptr)) {
    set_error("attn_decode: the rotary encoding is applied to all %d features of a head or to none, got %d", hd, rot);
    return ERR_UNSUPPORTED;
  }
  if (!aligned16(q) || !aligned16(k_pool) || !aligned16(v_pool) || !aligned16(out) || q_row_stride % 8 != 0) {
    set_error("attn_decode: q, k, v and out must be 16-byte aligned with a row stride in 16-byte units");
    return ERR_ALIGNMENT;
  }
  if (!in_block && exl3_attn_tokens_scratch_bytes(T, nh, hd, max_splits) > scratch_bytes) {
    set_error("attn_decode: scratch of %zu bytes is too small, need %zu", scratch_bytes,
              exl3_attn_tokens_scratch_bytes(T, nh, hd, max_splits));
    return ERR_SCRATCH;
  }
  static int sms = 0;
  if (!sms) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<64, 1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AD_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_kernel<128, 1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AD_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_kernel<64, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AD_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_kernel<128, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AD_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_kernel<64, 1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AD_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_kernel<128, 1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AD_SMEM);
    if (e != cudaSuccess) { set_error("attn_decode: cannot get %u bytes of shared memory: %s", AD_SMEM, cudaGetErrorString(e)); return (int)e; }
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms < 1) sms = 1;
  }
  // a stage is a page (heads of 64) or half a page (heads of 128): the copy's box has as many rows
  const int box_rows = hd == 64 ? 64 : 32;
  CUtensorMap map_k, map_v;
  int rc = ad_make_map(&map_k, k_pool, n_pool_rows, hd, box_rows);
  if (rc) return rc;
  rc = ad_make_map(&map_v, v_pool, n_pool_rows, hd, box_rows);
  if (rc) return rc;
  // one block per SM as soon as there is a chunk for each: the warps' equal shares then spread few chunks over all
  // SMs (and their memory pipes) instead of filling the warps of half of them
  const int groups = nkv * head_split;                     // groups of query heads worked on together
  if (max_splits > 1 && !in_block && (int64_t)T * groups > AD_COUNTER_SLOTS) {
    set_error("attn_decode: %d tokens x %d groups of heads exceed the %d merge counters", T, groups, AD_COUNTER_SLOTS);
    return ERR_UNSUPPORTED;
  }
  const int blocks = in_block ? T * (groups / twins) * (in_block == 2 ? 2 : 1)
                              : (int)std::min<int64_t>(sms, (int64_t)T * groups * max_splits);
  int* counters = max_splits > 1 && !in_block ? reinterpret_cast<int*>(scratch) : nullptr;
  float* records = max_splits > 1 && !in_block ? scratch + AD_COUNTER_SLOTS : nullptr;
#define EXL3_AD_LAUNCH(HD_, NC_, TW_)                                                                             \
  launch_pdl_clusters(attn_decode_kernel<HD_, NC_, TW_>, dim3(blocks), dim3((TW_ + 1) * AD_WARPS * 32),            \
             in_block == 2 ? 2u : 1u,                                                                              \
             (size_t)AD_SMEM, stream, map_k, map_v,                                                                \
             static_cast<const __nv_bfloat16*>(q), q_row_stride, static_cast<__nv_bfloat16*>(out), block_table,  \
             bt_stride, tok_pos, tok_seq, T, nh, groups, window, scale * 1.4426950408889634f, split_keys,        \
             max_splits, records, counters, inv_freq, inv_freq_lo, pos_scale, rot != 0 ? 1 : 0, write_new ? 1 : 0,            \
             static_cast<__nv_bfloat16*>(k_pool), static_cast<__nv_bfloat16*>(v_pool), head_split, in_block)
  const bool wide = nh / groups > 8;                       // more than one block of 8 query heads per group
  if (hd == 64) { if (wide) EXL3_AD_LAUNCH(64, 2, 1); else if (twins == 2) EXL3_AD_LAUNCH(64, 1, 2); else EXL3_AD_LAUNCH(64, 1, 1); }
  else { if (wide) EXL3_AD_LAUNCH(128, 2, 1); else if (twins == 2) EXL3_AD_LAUNCH(128, 1, 2); else EXL3_AD_LAUNCH(128, 1, 1); }
#undef EXL3_AD_LAUNCH
  return launch_status("attn_decode");
}
