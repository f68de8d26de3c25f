// Causal grouped-query attention of whole prompts over the paged cache on the
// 5th-generation tensor cores (heads of 64 or 128, bfloat16, pages of 64 keys).
//
// Same mathematics as attention_simt.cu (the
// reference's masked scaled-dot-product attention, src/model.cpp:539-548,
// 576-578).  A block owns 128 consecutive queries of one sequence and one head
// (or two such tiles, one after the other: see the kernel) and walks the key pages
// its queries may see:
//
//   warp 5     S = Q K^T as tcgen05.mma into one of two S buffers of 64 columns in tensor
//              memory, as soon as a page has landed and the buffer has been read: up to two
//              pages ahead of the softmax
//   warp 4     TMA copies of the Q tile and of K and V pages (straight from the paged
//              cache, 128B-swizzled) into a ring of stages, and O += P V as tcgen05.mma
//              (P read from tensor memory, two buffers of 32 columns; O in head_dim
//              columns) as soon as a P is handed over; the page that comes into a stage
//              next is asked for when the product that read the stage is done.
//              A head of 128 is two boxes of 64 features for every copy, two groups of
//              four instructions for S and two halves of O.  An instruction of 64 columns
//              holds its issuing thread for some 49 cycles when the SM's other block issues
//              none (measured: 47 cycles at least whatever the width, 64.5 at 128 columns,
//              128 at 256), about 100 when it does, and asking for a copy some hundred
//              more: with one warp for everything a page's issues and waits took as long
//              as its softmax, and each waited for the other.
//   warps 0-3  softmax: thread r owns query row r = TMEM lane r.  It reads its row
//              of S with tcgen05.ld (no shuffles: the whole row is in its
//              registers), masks, takes 2^(s * scale - m) with one multiply-add
//              and one ex2 per score, writes P as bfloat16 back into tensor memory
//              (the A operand of the second product is read from there), and at the
//              end reads O, divides by the row sum and stores 128 bytes.
//
// O is rescaled lazily: the maximum used for the exponentials only moves when a
// row's true maximum has grown by more than 2^8, so P stays below 256 and the
// accumulator in tensor memory is touched (tcgen05.ld / st) only then.
//
// Every mbarrier wait is bounded; a kernel that gives up records a code that
// exl3_attn_prefill_tc_status() returns, frees its tensor memory and exits.
#include "api.h"
#include "common.cuh"

#include <cuda.h>
#include <math.h>

namespace exl3 {

constexpr int FA_BQ = 128, FA_BK = 64;
constexpr int FA_THREADS = 160;                              // the four-blocks-an-SM kernel: softmax warps and one issuer
constexpr int FA_THREADS_MAIN = 192;                         // the kernel below: softmax warps, an MMA warp, a copy warp
constexpr int FA_KV_STAGES = 4;
// Tensor memory columns: S0 (64) | S1 (64) | O (head_dim) | P0 (32) | P1 (32); an allocation is a power of two.
__host__ __device__ constexpr int fa_tmem_cols(int hd) { return hd == 64 ? 256 : 512; }
__host__ __device__ constexpr uint32_t fa_q_bytes(int hd) { return FA_BQ * hd * 2; }
__host__ __device__ constexpr uint32_t fa_kv_bytes(int hd) { return FA_BK * hd * 2; }
__host__ __device__ constexpr uint32_t fa_smem(int hd) { return 2 * fa_q_bytes(hd) + 2 * FA_KV_STAGES * fa_kv_bytes(hd) + 1024 + 256; }
constexpr uint32_t FA_QBOX_BYTES = FA_BQ * 128, FA_KVBOX_BYTES = FA_BK * 128;   // a box of 64 features
constexpr uint64_t FA_WAIT_NS = 250000000ull;     // a wait gives up after a quarter of a second
constexpr float FA_RESCALE_STEP = 8.0f;           // in base-2 units

static __device__ int g_fa_error = 0;

__device__ inline uint32_t fa_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ inline void fa_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fa_smem_u32(bar)), "r"(count));
}
__device__ inline void fa_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fa_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ inline void fa_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fa_smem_u32(bar)) : "memory");
}
// A bounded wait: mbarrier.try_wait (which the hardware may hold for a while before it answers; a try that
// cannot succeed came back within a few cycles when measured) in a loop that looks at the clock after every
// try that failed and gives up FA_WAIT_NS after the first.
__device__ inline bool fa_mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = fa_smem_u32(bar);
  uint64_t t0 = 0;
  for (;;) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
    uint64_t now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (t0 == 0) t0 = now;
    else if (now - t0 > FA_WAIT_NS) return false;
  }
}
// One look at a phase: whether it has completed.
__device__ inline bool fa_mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(fa_smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ inline float fa_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ inline void fa_tma_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(fa_smem_u32(dst)), "l"(map), "r"(fa_smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ inline void fa_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void fa_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ inline void fa_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(fa_smem_u32(bar)) : "memory");
}
// Shared-memory operand descriptors (128B swizzle, version 1): K-major tiles have
// rows of 128 bytes in groups of 8 rows, 1024 bytes apart; the MN-major V tile
// has the same bytes, read as 8-key groups 1024 bytes apart.
__device__ inline uint64_t fa_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3fff) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16, D float32, A and B bfloat16, M = 128, N = 64; B K-major (S) or MN-major (PV)
constexpr uint32_t FA_IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t FA_IDESC_PV = FA_IDESC_S | (1u << 16);

__device__ inline void fa_umma(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// the same with the A operand in tensor memory (lanes = rows, two bfloat16 per column)
__device__ inline void fa_umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ inline void fa_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ inline void fa_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ inline void fa_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ inline void fa_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ inline float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ inline uint32_t fa_pack(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// What a block needs to know of a tile of 128 queries.
struct FaTile {
  int row0;        // the tile's first row of q and out
  int rows;        // its queries
  int p_first, p_last;   // their positions
  int page_lo;     // the first page they may see
  int n_pages;     // pages to walk
  const int* bt;   // the sequence's page table
};
__device__ inline FaTile fa_tile(int tile, const int* block_table, int bt_stride, const int* row_start,
                                 const int* row_pos0, const int* tile_seq, const int* tile_q0, int window) {
  FaTile t;
  const int b = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = row_start[b + 1] - row_start[b];
  t.row0 = row_start[b] + q0;
  t.rows = min(FA_BQ, n_new - q0);
  t.p_first = row_pos0[b] + q0;
  t.p_last = t.p_first + t.rows - 1;
  const int k_lo = (window > 0 && t.p_first - window + 1 > 0) ? t.p_first - window + 1 : 0;
  t.page_lo = k_lo / FA_BK;
  t.n_pages = t.p_last / FA_BK - t.page_lo + 1;
  t.bt = block_table + (int64_t)b * bt_stride;
  return t;
}

// fold = 0: block (head, y) owns tile y.  fold = 1: it owns tiles y and n_tiles - 1 - y of the caller's list
// (heaviest first), one after the other, so that all blocks have about the same number of pages to walk; the
// pages of both run through the same rings and buffers as one sequence of pages, the second tile's Q in a buffer
// of its own from the start, its first S products issued while the first tile's last softmax and epilogue run.
template <int FA_HD>
__global__ void __launch_bounds__(FA_THREADS_MAIN, FA_HD == 64 ? 2 : 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ block_table, int bt_stride, const int* __restrict__ row_start,
                       const int* __restrict__ row_pos0, const int* __restrict__ tile_seq,
                       const int* __restrict__ tile_q0, int n_tiles, int fold, int nh, int nkv, int window,
                       float scale_log2) {
  extern __shared__ unsigned char fa_smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int NB = FA_HD / 64;                             // boxes of 64 features (128-byte lines) in a head
  constexpr uint32_t FA_Q_BYTES = fa_q_bytes(FA_HD), FA_KV_BYTES = fa_kv_bytes(FA_HD);
  constexpr int FA_TMEM_COLS = fa_tmem_cols(FA_HD);
  unsigned char* sQ = base;                                  // [2 tiles][boxes][128][64] bf16
  unsigned char* sK = sQ + 2 * FA_Q_BYTES;                   // [stages][boxes][64][64]
  unsigned char* sV = sK + FA_KV_STAGES * FA_KV_BYTES;       // [stages][boxes][64][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + FA_KV_STAGES * FA_KV_BYTES);
  uint64_t* q_full = bars;                        // [2] Q tile landed
  uint64_t* kv_full = bars + 2;                   // [stages] K and V page landed
  uint64_t* kv_free = kv_full + FA_KV_STAGES;     // [stages] the products that read the stage are done
  uint64_t* s_full = kv_free + FA_KV_STAGES;      // [2] S buffer written by the tensor core
  uint64_t* s_free = s_full + 2;                  // [2] S buffer read by all 128 softmax threads
  uint64_t* p_full = s_free + 2;                  // [2] P buffer written by all 128 softmax threads
  uint64_t* pv_done = p_full + 2;                 // [2] O += P V of that P buffer finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the caller lists the tiles with the most keys to visit first
  const int head = blockIdx.x;                      // blocks start in this order: all heads of y = 0, then y = 1, ...
  const int g = head / (nh / nkv);
  const int other = n_tiles - 1 - (int)blockIdx.y;
  const int n_own = (fold && other > (int)blockIdx.y) ? 2 : 1;
  auto tile_of = [&](int w) {                       // the block's first (w = 0) or second tile
    return fa_tile(w ? other : (int)blockIdx.y, block_table, bt_stride, row_start, row_pos0, tile_seq, tile_q0, window);
  };

  if (threadIdx.x == 0) {
    fa_mbar_init(q_full, 1);
    fa_mbar_init(q_full + 1, 1);
    for (int i = 0; i < FA_KV_STAGES; ++i) {
      fa_mbar_init(kv_full + i, 1);
      fa_mbar_init(kv_free + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      fa_mbar_init(s_full + i, 1);
      fa_mbar_init(s_free + i, 128);
      fa_mbar_init(p_full + i, 128);
      fa_mbar_init(pv_done + i, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(fa_smem_u32(tmem_slot)), "r"(FA_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fa_fence_before();
  __syncthreads();
  fa_fence_after();
  // so far nothing was touched that another kernel writes; the next kernel in the stream may be set up meanwhile
  pdl_trigger();
  pdl_wait();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128;                  // columns: S0 0..63, S1 64..127, O from 128
  const uint32_t tmem_p = tmem_base + 128 + FA_HD;          // P0, then P1: 32 columns each (two bfloat16 per column)
  bool ok = true;

  if (warp == 4) {
    // ---- copies and the second product ---------------------------------------------------
    // The Q tiles and the first pages' K and V at once; then O += P_f V_f as soon as the softmax threads hand P_f
    // over, and, once that product is done with its stage of the ring, the copy of the page that comes into the
    // stage next.  This warp has most of a page's time to spare; the first product's warp has not (a copy asked
    // for there delayed S by more than it cost here).  Page numbers come 32 at a time, lane i holding the number of
    // page c0 + i of the block's walk, a batch ahead.
    const FaTile ta = tile_of(0), tb = n_own == 2 ? tile_of(1) : ta;
    const int n0 = ta.n_pages;
    const int n_total = n0 + (n_own == 2 ? tb.n_pages : 0);   // the block's pages, numbered through both tiles
    if (lane == 0) {
      for (int w = 0; w < n_own; ++w) {
        fa_mbar_expect_tx(q_full + w, FA_Q_BYTES);
#pragma unroll
        for (int x = 0; x < NB; ++x)
          fa_tma_2d(sQ + w * FA_Q_BYTES + x * FA_QBOX_BYTES, &map_q, q_full + w, head * FA_HD + 64 * x, w ? tb.row0 : ta.row0);
      }
    }
    auto numbers = [&](int c0) {                             // this lane's page number of the 32 from c0
      const int c = c0 + lane;
      if (c >= n_total) return 0;
      return c >= n0 ? tb.bt[tb.page_lo + c - n0] : ta.bt[ta.page_lo + c];
    };
    int pgs = numbers(0), pgs_next = numbers(32);
    int copied = 0;                                          // pages whose copies were asked for
    auto copy_next = [&]() {                                 // its stage is known to be free
      const int c = copied++;
      if ((c & 31) == 0 && c > 0) { pgs = pgs_next; pgs_next = numbers(c + 32); }
      const int st = c % FA_KV_STAGES;
      const int pg = __shfl_sync(0xffffffffu, pgs, c & 31);
      if (lane == 0) {
        fa_mbar_expect_tx(kv_full + st, 2 * FA_KV_BYTES);
#pragma unroll
        for (int x = 0; x < NB; ++x) {
          fa_tma_2d(sK + st * FA_KV_BYTES + x * FA_KVBOX_BYTES, &map_k, kv_full + st, 64 * x, (pg * nkv + g) * FA_BK);
          fa_tma_2d(sV + st * FA_KV_BYTES + x * FA_KVBOX_BYTES, &map_v, kv_full + st, 64 * x, (pg * nkv + g) * FA_BK);
        }
      }
      __syncwarp();
    };
    while (copied < FA_KV_STAGES && copied < n_total) copy_next();
    for (int f = 0; f < n_total && ok; ++f) {
      const int sb = f & 1, st = f % FA_KV_STAGES;
      if (!fa_mbar_wait(p_full + sb, (f >> 1) & 1)) { ok = false; break; }
      fa_fence_after();
      if (lane == 0) {
        // a tile's first product starts O afresh (the softmax threads hand over P only after they have read
        // the tile before out of O)
        const bool first = f == 0 || f == n0;
#pragma unroll
        for (int x = 0; x < NB; ++x) {                       // 64 features of O at a time
          const uint64_t db = fa_desc(fa_smem_u32(sV + st * FA_KV_BYTES + x * FA_KVBOX_BYTES));
#pragma unroll
          for (int k = 0; k < FA_BK / 16; ++k)              // 16 keys: 8 columns of P, 16 rows of V
            fa_umma_ts(tmem_o + 64 * x, tmem_p + sb * 32 + 8 * k, db + 128 * k, FA_IDESC_PV, (!first || k > 0) ? 1u : 0u);
        }
        fa_commit(pv_done + sb);
        fa_commit(kv_free + st);
      }
      __syncwarp();
      if (copied < n_total) {                                // page f + stages into the stage that page f leaves
        if (!fa_mbar_wait(kv_free + st, (f / FA_KV_STAGES) & 1)) { ok = false; break; }
        copy_next();
      }
    }
    if (!ok) {
      // a wait ran out: say so; the copies already asked for must land before the block's shared memory goes
      // away (when all is well the other product's warp has waited for every one of them)
      for (int u = max(0, copied - FA_KV_STAGES); u < copied; ++u)
        fa_mbar_wait(kv_full + u % FA_KV_STAGES, (u / FA_KV_STAGES) & 1);
      for (int w = 0; w < n_own; ++w) fa_mbar_wait(q_full + w, 0);
      if (lane == 0) atomicExch(&g_fa_error, 1);
    }
  } else if (warp == 5) {
    // ---- first product: S_f = Q K_f^T as soon as page f has landed and the softmax threads have read S_(f-2) out
    // of the buffer: up to two pages ahead of the softmax -------------------------------------
    const int n0 = tile_of(0).n_pages;
    const int n_total = n0 + (n_own == 2 ? tile_of(1).n_pages : 0);
    int q_seen = 0;                                          // Q tiles known to have landed
    for (int f = 0; f < n_total && ok; ++f) {
      const int sb = f & 1, st = f % FA_KV_STAGES;
      const int w = f >= n0 ? 1 : 0;
      if (q_seen <= w) {
        if (!fa_mbar_wait(q_full + w, 0)) { ok = false; break; }
        q_seen = w + 1;
      }
      if (!fa_mbar_wait(kv_full + st, (f / FA_KV_STAGES) & 1)) { ok = false; break; }
      if (f >= 2 && !fa_mbar_wait(s_free + sb, ((f >> 1) - 1) & 1)) { ok = false; break; }
      fa_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int x = 0; x < NB; ++x) {                       // 64 features of the sum at a time
          const uint64_t da = fa_desc(fa_smem_u32(sQ + w * FA_Q_BYTES + x * FA_QBOX_BYTES));
          const uint64_t db = fa_desc(fa_smem_u32(sK + st * FA_KV_BYTES + x * FA_KVBOX_BYTES));
#pragma unroll
          for (int k = 0; k < 4; ++k) fa_umma(tmem_base + sb * 64, da + 2 * k, db + 2 * k, FA_IDESC_S, (x | k) > 0);
        }
        fa_commit(s_full + sb);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) atomicExch(&g_fa_error, 3);
  } else {
    // ---- softmax and epilogue: thread r = query row r = TMEM lane r ---------------------
    const int r = threadIdx.x;                               // 0..127
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    int fb = 0;                                              // a tile's first page in the block's numbering
    for (int w = 0; w < n_own && ok; ++w) {
    const FaTile tw = tile_of(w);
    const int p_first = tw.p_first, p_last = tw.p_last, n_blocks = tw.n_pages, page_lo = tw.page_lo, rows = tw.rows;
    const int p = p_first + r;                               // this row's position
    float m_used = -INFINITY, l_run = 0.0f;
    // The row of S_f is asked for as soon as the row of P_(f-1) is on its way into tensor memory (the first of a
    // tile: here), so that the load's latency and the store's pass together.
    uint32_t sr[2][32];
    auto ask_s = [&](int f, bool there) -> bool {           // there: the barrier is known to have flipped
      const int st = f & 1;
      if (!there && !fa_mbar_wait(s_full + st, (f >> 1) & 1)) return false;
      fa_fence_after();
      fa_ld32(tmem_base + lane_addr + st * 64, sr[0]);
      fa_ld32(tmem_base + lane_addr + st * 64 + 32, sr[1]);
      return true;
    };
    ok = ask_s(fb, false);
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int f = fb + j;
      const int st = f & 1;
      fa_wait_ld();
      fa_fence_before();
      fa_mbar_arrive(s_free + st);
      // The two barriers this page still needs (the P buffer free again, the next S written) are looked at now:
      // both have almost always flipped a page ago, and the looks' trips to shared memory pass under the
      // arithmetic below instead of standing in front of the store of P and the load of S.
      const bool p_free = f < 2 || fa_mbar_test(pv_done + st, ((f - 2) >> 1) & 1);
      const bool s_there = j + 1 < n_blocks && fa_mbar_test(s_full + (st ^ 1), ((f + 1) >> 1) & 1);
      const int key0 = (page_lo + j) * FA_BK;
      const bool need_mask = (key0 + FA_BK - 1 > p_first) || (window > 0 && key0 <= p_last - window);
      // four independent chains for the maximum (and below for the sum): the row is long and
      // a single chain would make every step wait for the one before
      // masking without branches (one test per page decides whether the page needs it at all)
      if (need_mask) {
        const int lo_key = (window > 0) ? p - window : -1;    // keys <= lo_key are out of the window
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int key = key0 + h * 32 + c;
            const bool dead = (key > p) | (key <= lo_key);
            sr[h][c] = dead ? 0xff800000u : sr[h][c];         // -inf
          }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int c = 0; c < 32; c += 2)                      // two scores an instruction
          mx4[(c >> 1) & 3] = fa_max3(mx4[(c >> 1) & 3], __uint_as_float(sr[h][c]), __uint_as_float(sr[h][c + 1]));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= scale_log2;                                      // scale > 0: max and scale commute
      // lazy rescale: move the reference maximum only when it is far behind
      const bool grow = mx > m_used + FA_RESCALE_STEP || (m_used == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx : m_used;
        const float corr = (m_used == -INFINITY) ? 0.0f : fa_exp2(m_used - m_new);   // 1 for rows that keep theirs
        if (j > 0) {
          // every earlier product must have landed in O before it is rewritten
          if (!fa_mbar_wait(pv_done + (st ^ 1), ((f - 1) >> 1) & 1)) { ok = false; break; }
          fa_fence_after();
#pragma unroll
          for (int h2 = 0; h2 < FA_HD / 64; ++h2) {          // 64 columns at a time
            uint32_t o[2][32];
            fa_ld32(tmem_o + lane_addr + 64 * h2, o[0]);
            fa_ld32(tmem_o + lane_addr + 64 * h2 + 32, o[1]);
            fa_wait_ld();
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int c = 0; c < 32; ++c) o[h][c] = __float_as_uint(__uint_as_float(o[h][c]) * corr);
            fa_st32(tmem_o + lane_addr + 64 * h2, o[0]);
            fa_st32(tmem_o + lane_addr + 64 * h2 + 32, o[1]);
          }
          fa_wait_st();
          fa_fence_before();
        }
        l_run *= corr;
        m_used = m_new;
      }
      const float mref = (m_used == -INFINITY) ? 0.0f : m_used;
      // the P buffer of two pages ago must have been consumed
      if (!p_free && !fa_mbar_wait(pv_done + st, ((f - 2) >> 1) & 1)) { ok = false; break; }
      uint32_t pw[32];
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int c = 0; c < 32; ++c) {                         // two keys per column
        const float e0 = fa_exp2(fmaf(__uint_as_float(sr[(2 * c) >> 5][(2 * c) & 31]), scale_log2, -mref));
        const float e1 = fa_exp2(fmaf(__uint_as_float(sr[(2 * c + 1) >> 5][(2 * c + 1) & 31]), scale_log2, -mref));
        sum4[c & 3] += e0 + e1;
        pw[c] = fa_pack(e0, e1);
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l_run += sum;
      fa_st32(tmem_p + lane_addr + st * 32, pw);
      if (j + 1 < n_blocks && !ask_s(f + 1, s_there)) ok = false;   // the tile's next row of S while P is being stored
      fa_wait_st();
      fa_fence_before();
      fa_mbar_arrive(p_full + st);
    }
    if (ok) {
      // last product done -> O complete
      const int fl = fb + n_blocks - 1;
      ok = fa_mbar_wait(pv_done + (fl & 1), (fl >> 1) & 1);
      if (ok) {
        fa_fence_after();
        const float inv = 1.0f / l_run;
        __nv_bfloat16* dst = out + ((int64_t)(tw.row0 + r) * nh + head) * FA_HD;
#pragma unroll
        for (int h2 = 0; h2 < FA_HD / 64; ++h2) {            // 64 columns at a time (every thread reads: the load is the warp's)
          uint32_t o[2][32];
          fa_ld32(tmem_o + lane_addr + 64 * h2, o[0]);
          fa_ld32(tmem_o + lane_addr + 64 * h2 + 32, o[1]);
          fa_wait_ld();
          if (r < rows) {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              uint4 wd;
              const int c = ch * 8;
              wd.x = fa_pack(__uint_as_float(o[c >> 5][(c & 31) + 0]) * inv, __uint_as_float(o[c >> 5][(c & 31) + 1]) * inv);
              wd.y = fa_pack(__uint_as_float(o[c >> 5][(c & 31) + 2]) * inv, __uint_as_float(o[c >> 5][(c & 31) + 3]) * inv);
              wd.z = fa_pack(__uint_as_float(o[c >> 5][(c & 31) + 4]) * inv, __uint_as_float(o[c >> 5][(c & 31) + 5]) * inv);
              wd.w = fa_pack(__uint_as_float(o[c >> 5][(c & 31) + 6]) * inv, __uint_as_float(o[c >> 5][(c & 31) + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + 64 * h2 + c) = wd;
            }
          }
        }
        fa_fence_before();                                 // O is read: the next tile's first product may write it
      }
    }
    fb += n_blocks;
    }
    if (!ok) fa_wait_ld();                                   // a row of S may still be on its way
    if (!ok && lane == 0) atomicExch(&g_fa_error, 2);
  }

  fa_fence_before();
  __syncthreads();
  fa_fence_after();
  if (warp == 4)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(FA_TMEM_COLS) : "memory");
}


// ---- heads of 64: four blocks per SM ---------------------------------------------------------------
// What bounds the kernel above is the chain of fixed latencies inside one page of a row's softmax, with two warps
// per scheduler to hide it.  This variant trades the overlap inside a block (one S buffer instead of two, P written
// over S, a ring of two pages) for blocks: 128 columns of tensor memory, 49 KB of shared memory and at most 102
// registers a thread let four blocks share an SM, sixteen softmax warps instead of eight.  A block alone is
// slower (1.64 against 1.53 us a page), so the variant is used when the blocks do not all fit the GPU at once
// (more than four per SM): 452 against 530 us at 8,192 tokens with 36 heads, 84 against 96 us at 3,072, 117 against
// 142 us for 24 prompts of 16 to 2,048 tokens with 16 heads; at 2,048 tokens, where one wave of blocks runs and the
// heaviest tile's 32 pages are the kernel's length, the kernel above stays (48.7 against 52.6 us).  Same
// arithmetic in the same order per row: the two give the same numbers bit for bit.
constexpr int F4_STAGES = 2;
constexpr uint32_t F4_SMEM = fa_q_bytes(64) + 2 * F4_STAGES * fa_kv_bytes(64) + 1024 + 128;

__global__ void __launch_bounds__(FA_THREADS, 4)
attn_prefill_tc4_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ block_table, int bt_stride, const int* __restrict__ row_start,
                        const int* __restrict__ row_pos0, const int* __restrict__ tile_seq,
                        const int* __restrict__ tile_q0, int nh, int nkv, int window, float scale_log2) {
  extern __shared__ unsigned char fa_smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr uint32_t QB = fa_q_bytes(64), KVB = fa_kv_bytes(64);
  unsigned char* sQ = base;
  unsigned char* sK = sQ + QB;
  unsigned char* sV = sK + F4_STAGES * KVB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + F4_STAGES * KVB);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                   // [2]
  uint64_t* kv_free = kv_full + F4_STAGES;        // [2]
  uint64_t* s_full = kv_free + F4_STAGES;         // S written by the tensor core
  uint64_t* p_full = s_full + 1;                  // P written over S by all 128 softmax threads
  uint64_t* pv_done = p_full + 1;                 // O += P V finished: the S columns are free again
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x, tile = blockIdx.y;
  const int b = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = row_start[b + 1] - row_start[b];
  const int pos0 = row_pos0[b];
  const int g = head / (nh / nkv);
  const int rows = min(FA_BQ, n_new - q0);
  const int p_first = pos0 + q0, p_last = pos0 + q0 + rows - 1;
  const int k_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  const int page_lo = k_lo / FA_BK, page_hi = p_last / FA_BK;
  const int n_blocks = page_hi - page_lo + 1;
  const int* bt = block_table + (int64_t)b * bt_stride;

  if (threadIdx.x == 0) {
    fa_mbar_init(q_full, 1);
    for (int i = 0; i < F4_STAGES; ++i) { fa_mbar_init(kv_full + i, 1); fa_mbar_init(kv_free + i, 1); }
    fa_mbar_init(s_full, 1);
    fa_mbar_init(p_full, 128);
    fa_mbar_init(pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(fa_smem_u32(tmem_slot)), "r"(128) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fa_fence_before();
  __syncthreads();
  fa_fence_after();
  // so far nothing was touched that another kernel writes; the next kernel in the stream may be set up meanwhile
  pdl_trigger();
  pdl_wait();
  const uint32_t tmem_base = *tmem_slot;                    // columns: S 0..63 (P over 0..31), O 64..127
  const uint32_t tmem_o = tmem_base + 64;
  bool ok = true;

  if (warp == 4) {
    // ---- issuer: TMA and MMA -----------------------------------------------------------
    if (lane == 0) {
      fa_mbar_expect_tx(q_full, QB);
      fa_tma_2d(sQ, &map_q, q_full, head * 64, row_start[b] + q0);
    }
    auto load_kv = [&](int j) {
      const int st = j % F4_STAGES;
      const int pg = bt[page_lo + j];
      if (lane == 0) {
        fa_mbar_expect_tx(kv_full + st, 2 * KVB);
        fa_tma_2d(sK + st * KVB, &map_k, kv_full + st, 0, (pg * nkv + g) * FA_BK);
        fa_tma_2d(sV + st * KVB, &map_v, kv_full + st, 0, (pg * nkv + g) * FA_BK);
      }
    };
    for (int j = 0; j < F4_STAGES && j < n_blocks; ++j) load_kv(j);
    ok = fa_mbar_wait(q_full, 0);
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int st = j % F4_STAGES;
      if (!fa_mbar_wait(kv_full + st, (j / F4_STAGES) & 1)) { ok = false; break; }
      // S_j goes where P of page j - 1 still is until that page's product is done
      if (j > 0 && !fa_mbar_wait(pv_done, (j - 1) & 1)) { ok = false; break; }
      fa_fence_after();
      if (lane == 0) {
        const uint64_t da = fa_desc(fa_smem_u32(sQ));
        const uint64_t db = fa_desc(fa_smem_u32(sK + st * KVB));
#pragma unroll
        for (int k = 0; k < 4; ++k) fa_umma(tmem_base, da + 2 * k, db + 2 * k, FA_IDESC_S, k > 0);
        fa_commit(s_full);
      }
      __syncwarp();
      // the stage of page j - 1 is free (its product is done): the page after next goes there
      if (j >= 1 && j + 1 < n_blocks) load_kv(j + 1);
      if (!fa_mbar_wait(p_full, j & 1)) { ok = false; break; }
      fa_fence_after();
      if (lane == 0) {
        const uint64_t db = fa_desc(fa_smem_u32(sV + st * KVB));
#pragma unroll
        for (int k = 0; k < FA_BK / 16; ++k)
          fa_umma_ts(tmem_o, tmem_base + 8 * k, db + 128 * k, FA_IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
        fa_commit(pv_done);
      }
      __syncwarp();
    }
    if (!ok) {
      for (int j = max(0, n_blocks - F4_STAGES); j < n_blocks; ++j) fa_mbar_wait(kv_full + j % F4_STAGES, (j / F4_STAGES) & 1);
      if (lane == 0) atomicExch(&g_fa_error, 1);
    }
  } else {
    // ---- softmax and epilogue: thread r = query row r = TMEM lane r ---------------------
    const int r = threadIdx.x;
    const int p = p_first + r;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float m_used = -INFINITY, l_run = 0.0f;
    for (int j = 0; j < n_blocks && ok; ++j) {
      if (!fa_mbar_wait(s_full, j & 1)) { ok = false; break; }
      fa_fence_after();
      uint32_t sr[2][32];
      fa_ld32(tmem_base + lane_addr, sr[0]);
      fa_ld32(tmem_base + lane_addr + 32, sr[1]);
      fa_wait_ld();
      const int key0 = (page_lo + j) * FA_BK;
      const bool need_mask = (key0 + FA_BK - 1 > p_first) || (window > 0 && key0 <= p_last - window);
      if (need_mask) {
        const int lo_key = (window > 0) ? p - window : -1;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int key = key0 + h * 32 + c;
            const bool dead = (key > p) | (key <= lo_key);
            sr[h][c] = dead ? 0xff800000u : sr[h][c];
          }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int c = 0; c < 32; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[h][c]));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= scale_log2;
      const bool grow = mx > m_used + FA_RESCALE_STEP || (m_used == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx : m_used;
        const float corr = (m_used == -INFINITY) ? 0.0f : fa_exp2(m_used - m_new);
        if (j > 0) {
          // the product of page j - 1 is in O: S_j was issued after it was done.  16 columns at a time: the
          // row of scores stays in its registers meanwhile
#pragma unroll 1
          for (int c0 = 0; c0 < 64; c0 += 16) {
            uint32_t o[16];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                         : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3]), "=r"(o[4]), "=r"(o[5]), "=r"(o[6]), "=r"(o[7]),
                           "=r"(o[8]), "=r"(o[9]), "=r"(o[10]), "=r"(o[11]), "=r"(o[12]), "=r"(o[13]), "=r"(o[14]), "=r"(o[15])
                         : "r"(tmem_o + lane_addr + c0));
            fa_wait_ld();
#pragma unroll
            for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
            asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                         ::"r"(tmem_o + lane_addr + c0), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]),
                           "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15]) : "memory");
          }
          fa_wait_st();
        }
        l_run *= corr;
        m_used = m_new;
      }
      const float mref = (m_used == -INFINITY) ? 0.0f : m_used;
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int c = 0; c < 32; ++c) {                         // two keys per column, written over the scores' registers
        const float e0 = fa_exp2(fmaf(__uint_as_float(sr[(2 * c) >> 5][(2 * c) & 31]), scale_log2, -mref));
        const float e1 = fa_exp2(fmaf(__uint_as_float(sr[(2 * c + 1) >> 5][(2 * c + 1) & 31]), scale_log2, -mref));
        sum4[c & 3] += e0 + e1;
        sr[0][c] = fa_pack(e0, e1);
      }
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      fa_st32(tmem_base + lane_addr, sr[0]);
      fa_wait_st();
      fa_fence_before();
      fa_mbar_arrive(p_full);
    }
    if (ok) {
      const int jl = n_blocks - 1;
      ok = fa_mbar_wait(pv_done, jl & 1);
      if (ok) {
        fa_fence_after();
        const float inv = 1.0f / l_run;
        __nv_bfloat16* dst = out + ((int64_t)(row_start[b] + q0 + r) * nh + head) * 64;
#pragma unroll 1
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t o[32];
          fa_ld32(tmem_o + lane_addr + c0, o);
          fa_wait_ld();
          if (r < rows) {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              uint4 w;
              const int c = ch * 8;
              w.x = fa_pack(__uint_as_float(o[c + 0]) * inv, __uint_as_float(o[c + 1]) * inv);
              w.y = fa_pack(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
              w.z = fa_pack(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
              w.w = fa_pack(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c0 + c) = w;
            }
          }
        }
      }
    }
    if (!ok && lane == 0) atomicExch(&g_fa_error, 2);
  }

  fa_fence_before();
  __syncthreads();
  fa_fence_after();
  if (warp == 4)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128) : "memory");
}

// ---- host side --------------------------------------------------------------------------

typedef CUresult (*FaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static FaEncodeFn fa_encode_fn() {
  static FaEncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<FaEncodeFn>(p);
  }();
  return fn;
}
// [rows, cols] bfloat16 with a row pitch in elements; boxes of box_rows x 64 columns, 128B swizzle.
static int fa_make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t pitch, int box_rows) {
  FaEncodeFn fn = fa_encode_fn();
  if (!fn) { set_error("attn_prefill_tc: the driver has no cuTensorMapEncodeTiled"); return ERR_UNSUPPORTED; }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("attn_prefill_tc: cuTensorMapEncodeTiled failed with %d", (int)r); return ERR_BAD_ARGUMENT; }
  return 0;
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_attn_prefill_tc_supported(int dtype, int hd, int page) {
  return dtype == DT_BF16 && (hd == 64 || hd == 128) && page == FA_BK;
}
extern "C" int exl3_attn_prefill_tc_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_fa_error, sizeof(int));
  if (v) { int z = 0; cudaMemcpyToSymbol(g_fa_error, &z, sizeof(int)); }
  return v;
}

// q: rows of the fused q|k|v buffer (row stride q_row_stride elements, T rows in all); tiles of 128 queries.
// n_pool_rows = pages * kv_heads * 64 rows of head_dim in each of k_pool and v_pool.
extern "C" int exl3_attn_prefill_tc(const void* q, int64_t q_row_stride, int T, void* out, const void* k_pool,
                                    const void* v_pool, int64_t n_pool_rows, const int* block_table, int bt_stride,
                                    const int* row_start, const int* row_pos0, const int* tile_seq,
                                    const int* tile_q0, int n_tiles, int nh, int nkv, int hd, int page, int window,
                                    float scale, int variant, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  if (!exl3_attn_prefill_tc_supported(DT_BF16, hd, page)) {
    set_error("attn_prefill_tc: needs bfloat16, head_dim 64 or 128 and pages of 64, got head_dim %d page %d", hd, page);
    return ERR_UNSUPPORTED;
  }
  if (variant < 0 || variant > 3 || (variant == 2 && hd != 64)) {
    set_error("attn_prefill_tc: variant is 0 (chosen), 1 (a tile a block), 2 (four blocks an SM, heads of 64) or 3 (two tiles a block), got %d", variant);
    return ERR_BAD_ARGUMENT;
  }
  if (n_tiles < 0 || T < 1 || nh < 1 || nkv < 1 || nh % nkv != 0 || n_tiles > 65535 || window < 0 || q_row_stride % 8 != 0) {
    set_error("attn_prefill_tc: bad sizes tiles=%d T=%d heads=%d kv_heads=%d window=%d", n_tiles, T, nh, nkv, window);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(q) || !aligned16(k_pool) || !aligned16(v_pool) || !aligned16(out)) {
    set_error("attn_prefill_tc: q, k, v and out must be 16-byte aligned");
    return ERR_ALIGNMENT;
  }
  static bool configured = false;
  static int sms = 148;
  if (!configured) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms < 1) sms = 148;
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F4_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_smem(64));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_smem(128));
    if (e != cudaSuccess) { set_error("attn_prefill_tc: cannot get %u bytes of shared memory: %s", fa_smem(128), cudaGetErrorString(e)); return (int)e; }
    configured = true;
  }
  CUtensorMap map_q, map_k, map_v;
  int rc = fa_make_map(&map_q, q, T, (int64_t)nh * hd, q_row_stride, FA_BQ);
  if (rc) return rc;
  rc = fa_make_map(&map_k, k_pool, n_pool_rows, hd, hd, FA_BK);
  if (rc) return rc;
  rc = fa_make_map(&map_v, v_pool, n_pool_rows, hd, hd, FA_BK);
  if (rc) return rc;
  // Four blocks an SM when there are more blocks than that holds at once.  Two tiles a block (the heaviest with
  // the lightest, and so on) when a tile a block would need a second round of blocks and two tiles a block need
  // none: then every block walks about the same number of pages and the kernel ends with all of them.
  const int64_t blocks = (int64_t)n_tiles * nh, at_once = (int64_t)sms * (hd == 64 ? 2 : 1);
  const bool four = hd == 64 && (variant == 2 || (variant == 0 && blocks > 4 * (int64_t)sms));
  const int fold = (variant == 3 || (variant == 0 && !four && blocks > at_once && (int64_t)((n_tiles + 1) / 2) * nh <= at_once)) ? 1 : 0;
  dim3 grid(nh, fold ? (n_tiles + 1) / 2 : n_tiles);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  const float scale_log2 = scale * 1.4426950408889634f;
  if (four)
    launch_pdl(attn_prefill_tc4_kernel, grid, dim3(FA_THREADS), F4_SMEM, stream, map_q, map_k, map_v, o, block_table,
               bt_stride, row_start, row_pos0, tile_seq, tile_q0, nh, nkv, window, scale_log2);
  else if (hd == 64)
    launch_pdl(attn_prefill_tc_kernel<64>, grid, dim3(FA_THREADS_MAIN), fa_smem(64), stream, map_q, map_k, map_v, o,
               block_table, bt_stride, row_start, row_pos0, tile_seq, tile_q0, n_tiles, fold, nh, nkv, window, scale_log2);
  else
    launch_pdl(attn_prefill_tc_kernel<128>, grid, dim3(FA_THREADS_MAIN), fa_smem(128), stream, map_q, map_k, map_v, o,
               block_table, bt_stride, row_start, row_pos0, tile_seq, tile_q0, n_tiles, fold, nh, nkv, window, scale_log2);
  return launch_status("attn_prefill_tc");
}
