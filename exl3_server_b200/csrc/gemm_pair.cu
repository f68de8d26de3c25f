// Projections of many rows (prompts) on the 5th-generation tensor cores, two blocks of a cluster as one tensor core:
//   y[M,N] = x[M,K] . w[N,K]^T (+ bias), bfloat16 operands, float32 accumulation in tensor memory
// In the reference these are library matmuls with separate element-wise ops around them (src/model.cpp:549,
// 583-586, 600-611).
//
// A pair of blocks (a cluster of two, on two neighbouring SMs) works on one tile of 256 x 256 outputs with
// tcgen05.mma.cta_group::2 (M 256, N 256, K 16): each block copies its 128 rows of x and its 128 rows of w into its
// own shared memory (16 KB + 16 KB per 64 of K, a ring of five stages), the pair's even block issues the
// instructions, which read both blocks' shared memory, and each block finds its 128 rows of the accumulator in its
// own tensor memory.  Per flop a block copies and reads two thirds of what a block that works alone on 128 x 256
// does; that is what lets the tensor pipe run without waiting for shared memory.
//
//   warp 0    TMA producer (both blocks): cp.async.bulk.tensor tiles, their bytes counted on the even block's
//             mbarrier; no multicast, every block copies what it needs itself
//   warp 1    even block: one thread issues the MMAs; tcgen05.commit frees ring stages in both blocks and hands
//             accumulators to both blocks' epilogues.  Both blocks: allocates and frees the tensor memory
//   warps 2-  epilogue (both blocks; eight warps, four with the residual epilogue): thread = row; 64 accumulator
//             columns at a time from tensor memory, results into 128B-swizzled staging tiles of 32 rows x 128
//             bytes, which TMA stores write out (clipped at the matrix's edges), so that no thread stores a
//             row-strided sliver itself
// Two accumulators (2 x 256 of the 512 columns) let the epilogue of one tile overlap the products of the next.
// Pairs are persistent; tiles go round-robin over them, M fastest, so that pairs that run together share w in L2.
//
// Input: x, or a norm's output in two pieces (x_raw = h * w_norm and per-row pieces of sum(h^2)): the accumulator is
// multiplied by k = rsqrt(sum / width + eps) per row.
// Epilogues: 0 y bfloat16; 1 silu(gate) * up for a weight whose rows are 8 gate rows, the 8 up rows of the same
// features, and so on (y is N/2 wide); 2 the output times rho is added to the float32 residual h in place, and the
// next norm's pieces are left: x_raw = h * w_norm and, per row and tile of 256 columns, sum(h^2).  For 2 the residual
// does not wait for the epilogue: while the tensor core is busy with earlier tiles, the epilogue warps bring the
// tile of h into the accumulator itself (TMA to shared memory, divided by rho * k, tcgen05.st), the products are
// added on top of it, and the epilogue only multiplies by rho * k, adds rho * bias and writes.  (The product is
// therefore not rounded to bfloat16 before it is added, as it is where the addition is a separate step.)
//
// Epilogue 3 is the q/k/v projection of heads of 64: the output, rounded to bfloat16 as the plain epilogue would
// store it, gets the half-split rotary encoding (queries and keys; a row's sines and cosines are computed once per
// tile, while the products run), the queries go to y, and the keys and values go straight to the token's place in
// the paged cache: as one TMA store where a warp's 32 rows are 32 consecutive places of one page, with 16-byte
// stores otherwise.  The key and value columns of y are not written.
//
// Every wait on an mbarrier is bounded: when one runs out the kernel records a code, leaves its loops, waits
// (bounded) for the copies it may have in flight, meets its partner at the cluster barrier that every path reaches,
// frees its tensor memory and returns; exl3_gemm_pair_status() reads the code.
#include "api.h"
#include "tcgen05.cuh"

#include <cuda.h>

namespace exl3 {

using namespace tc5;

constexpr int GP_BM = 256, GP_BN = 256, GP_BK = 64;
// Epilogue warps: four (one per 32 lanes of tensor memory), or eight, two per 32 lanes with half of the columns each.
__host__ __device__ constexpr int gp_epi_warps(int epi) { return epi >= 2 ? 4 : 8; }
__host__ __device__ constexpr int gp_threads(int epi) { return 64 + 32 * gp_epi_warps(epi); }
constexpr uint32_t GP_STAGE_A = 128 * GP_BK * 2, GP_STAGE_B = 128 * GP_BK * 2;       // per block
constexpr uint32_t GP_BOX = 32 * 128;                                                  // a staging tile: 32 rows x 128 bytes
__host__ __device__ constexpr int gp_stages(int) { return 5; }
__host__ __device__ constexpr int gp_boxes(int epi) { return epi == 2 ? 4 : 2; }       // staging tiles per epilogue warp
__host__ __device__ constexpr uint32_t gp_smem(int epi) {
  return 1024 /* alignment */ + gp_stages(epi) * (GP_STAGE_A + GP_STAGE_B) + gp_epi_warps(epi) * gp_boxes(epi) * GP_BOX +
         GP_BN * 4 /* norm weights */ + GP_BN * 2 /* bias */ + 256 /* barriers */;
}
constexpr uint32_t GP_IDESC = idesc_bf16(GP_BM, GP_BN);

static __device__ int g_gp_error = 0;

// Barrier 1 over the THREADS epilogue threads, returning whether the predicate held for all of them.
template <int THREADS> __device__ inline bool gp_epilogue_all(bool pred) {
  int r;
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.s32 p, %1, 0;\n\tbar.red.and.pred q, 1, %2, p;\n\tselp.s32 %0, 1, 0, q;\n\t}"
               : "=r"(r) : "r"((int)pred), "n"(THREADS) : "memory");
  return r != 0;
}
__device__ inline void gp_tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ inline uint32_t gp_pack(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// 16 bytes number j (0..7) of row r of a 128B-swizzled staging tile.
__device__ inline uint4* gp_box_chunk(unsigned char* box, int r, int j) {
  return reinterpret_cast<uint4*>(box + r * 128 + ((j ^ (r & 7)) << 4));
}

struct PairArgs {
  const __nv_bfloat16* bias;
  int M, N, K;
  const float* ss_in;        // [rows >= M, ss_blocks] or null
  int ss_blocks;
  float eps, width;
  float rho;
  const void* norm_w;        // [N], float32 or bfloat16
  int norm_w_f32;
  float* ss_out;             // [M, tiles of 256 columns]
  // epilogue 3
  const int* tok_pos;        // [M] position of each row's token
  const int* tok_seq;        // [M] its row of the block table
  const int* block_table;
  int bt_stride;
  const float* inv_freq;     // [32] rotary frequencies, or null for no rotation
  const float* inv_freq_lo;  // what float32 lost of them, or null
  float pos_scale;
  int nh, nkv;               // query and key/value heads of 64
  int write_kv;
  __nv_bfloat16* k_pool;     // [pages, nkv, 64, 64]
  __nv_bfloat16* v_pool;
};

template <int EPI>
__global__ void __launch_bounds__(gp_threads(EPI), 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_y,      // y (0, 1) or x_raw (2): bfloat16, boxes of 64 columns
                 const __grid_constant__ CUtensorMap map_h,      // 2: the float32 residual, boxes of 32 columns
                 const __grid_constant__ CUtensorMap map_k,      // 3: the key and the value pool as rows of 64 features,
                 const __grid_constant__ CUtensorMap map_v,      //    boxes of 32 rows
                 const PairArgs a) {
  constexpr int STAGES = gp_stages(EPI), BOXES = gp_boxes(EPI), EPI_WARPS = gp_epi_warps(EPI), EPI_THREADS = 32 * EPI_WARPS;
  extern __shared__ unsigned char gp_smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gp_smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = base;
  unsigned char* sB = base + STAGES * GP_STAGE_A;
  unsigned char* boxes = base + STAGES * (GP_STAGE_A + GP_STAGE_B);       // [EPI_WARPS][BOXES] staging tiles
  float* s_normw = reinterpret_cast<float*>(boxes + EPI_WARPS * BOXES * GP_BOX);
  __nv_bfloat16* s_bias = reinterpret_cast<__nv_bfloat16*>(s_normw + GP_BN);
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + GP_BN);
  uint64_t* full = bars;                       // [STAGES] even block only: both blocks' copies landed
  uint64_t* empty = bars + STAGES;             // [STAGES] each block: the MMAs that read the stage are done
  uint64_t* acc_full = bars + 2 * STAGES;      // [2] each block: accumulator complete
  uint64_t* acc_empty = acc_full + 2;          // [2] even block only: both blocks' epilogues are done with it
  uint64_t* hbar = acc_empty + 2;              // [4 warps][4] epilogue 2: a tile of h landed in a staging tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(hbar + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();        // 0: issues the MMAs
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  if (threadIdx.x == 0) {
    prefetch_map(&map_x);
    prefetch_map(&map_w);
    prefetch_map(&map_y);
    if (EPI == 2) prefetch_map(&map_h);
    if (EPI == 3) { prefetch_map(&map_k); prefetch_map(&map_v); }
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 2 * EPI_WARPS); }
    for (int i = 0; i < 16; ++i) mbar_init(hbar + i, 1);
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc_pair<512>(tmem_slot);
  fence_before();
  cluster_sync_all();                          // both blocks' barriers exist before either signals the other's
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything so far touched nothing that another kernel writes; from here on x, h and the norm's pieces are read
  // and results written.  The next kernel in the stream may be set up meanwhile.
  pdl_trigger();
  pdl_wait();

  const int n_m = (a.M + GP_BM - 1) / GP_BM, n_n = (a.N + GP_BN - 1) / GP_BN;
  const int n_tiles = n_m * n_n, kblocks = (a.K + GP_BK - 1) / GP_BK;
  // 2, when no pair has a second tile: the second accumulator is free, so the residual goes there while the products
  // start from zero in the first at once, and the epilogue adds the two.  (With several tiles per pair both
  // accumulators are in use in turn, and the residual goes into the accumulator before the tile's products.)
  const bool beside = EPI == 2 && n_tiles <= n_pairs;
  bool ok = true;

  if (warp == 0) {
    // ---- producer: this block's halves of the pair's tiles ---------------------------------------------
    uint32_t it = 0;
    for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
      const int m0 = (tile % n_m) * GP_BM + (int)rank * 128, n0 = (tile / n_m) * GP_BN + (int)rank * 128;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(empty + s, ((it / STAGES) & 1) ^ 1)) { ok = false; break; }
        if (lane == 0) {
          const uint32_t bar = cluster_addr(full + s, 0);
          if (rank == 0) mbar_expect_tx(full + s, 2 * (GP_STAGE_A + GP_STAGE_B));
          tma_load_2d_pair(sA + s * GP_STAGE_A, &map_x, bar, kb * GP_BK, m0);
          tma_load_2d_pair(sB + s * GP_STAGE_B, &map_w, bar, kb * GP_BK, n0);
        }
        __syncwarp();
      }
    }
    if (!ok) {
      if (lane == 0) atomicExch(&g_gp_error, 1);
      // Copies still in flight must land before either block's shared memory goes away.  Their bytes are counted
      // on the even block's barriers: it waits for the last stages it armed, and the partner stays until the
      // cluster barrier at the end, which the even block reaches after these waits.
      if (rank == 0)
        for (uint32_t back = 1; back <= (uint32_t)STAGES && back <= it; ++back) {
          const uint32_t j = it - back;
          mbar_wait(full + (j % STAGES), (j / STAGES) & 1);
        }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (even block) ----------------------------------------------------------------------------
    if (rank == 0) {
      uint32_t it = 0, tcount = 0;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++tcount) {
        const uint32_t buf = tcount & 1;
        // 0, 1: an accumulator is free from the start and after each epilogue; 2: it is ready when the epilogue
        // warps have put the tile's residual into it
        if (!beside && !mbar_wait(acc_empty + buf, ((tcount >> 1) & 1) ^ (EPI == 2 ? 0u : 1u))) { ok = false; break; }
        fence_after();
        const uint32_t d_tmem = tmem_base + buf * GP_BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full + s, (it / STAGES) & 1)) { ok = false; break; }
          fence_after();
          if (lane == 0) {
            const uint64_t da = smem_desc_k128(smem_u32(sA + s * GP_STAGE_A));
            const uint64_t db = smem_desc_k128(smem_u32(sB + s * GP_STAGE_B));
#pragma unroll
            for (int k = 0; k < GP_BK / 16; ++k)
              mma_ss_pair(d_tmem, da + 2 * k, db + 2 * k, GP_IDESC, ((EPI == 2 && !beside) || kb > 0 || k > 0) ? 1u : 0u);
            mma_commit_pair(empty + s);
          }
          __syncwarp();
        }
        if (!ok) break;
        if (lane == 0) mma_commit_pair(acc_full + buf);
        __syncwarp();
      }
      if (!ok && lane == 0) atomicExch(&g_gp_error, 2);
    }
  } else {
    // ---- epilogue: thread = row of this block's 128 -----------------------------------------------------------
    const int q = warp & 3;                               // the 32 TMEM lanes this warp may read
    const int t = (warp - 2) * 32 + lane;
    // with eight warps, warps 2-5 take the tile's columns 0-127 and warps 6-9 the columns 128-255
    const int s_lo = EPI_WARPS == 8 ? ((warp - 2) >> 2) * 2 : 0, s_hi = s_lo + (EPI_WARPS == 8 ? 2 : 4);
    unsigned char* my_boxes = boxes + (warp - 2) * BOXES * GP_BOX;
    uint64_t* my_hbar = hbar + q * 4;
    const uint32_t acc_empty_addr[2] = {cluster_addr(acc_empty, 0), cluster_addr(acc_empty + 1, 0)};
    const uint32_t lane_taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t n_store = 0;                                 // 0, 1: staging tiles stored so far (they alternate)
    uint32_t n_hload = 0;                                 // 2: tiles of h loaded so far (four staging tiles in turn)

    // k of a row: what its accumulator is multiplied by
    auto row_factor = [&](int row) {
      float k = 1.0f;
      if (a.ss_in && row < a.M) {
        float ss = 0.0f;
        for (int j = 0; j < a.ss_blocks; ++j) ss += __ldcg(a.ss_in + (int64_t)row * a.ss_blocks + j);
        k = rsqrtf(ss / a.width + a.eps);
      }
      return k;
    };
    // 2: this warp's 32 rows of a tile of h into accumulator `buf`: divided by rho * k, and the accumulator is then
    // handed to the MMA issuer; or as they are, beside the products.  False when a wait ran out.
    auto preload = [&](int tile, uint32_t buf) -> bool {
      const int row0 = (tile % n_m) * GP_BM + (int)rank * 128 + q * 32, n0 = (tile / n_m) * GP_BN;
      const float inv = beside ? 1.0f : 1.0f / (a.rho * row_factor(row0 + lane));
      if (lane == 0) tma_store_wait_read<0>();            // the last epilogue's stores have read the staging tiles
      __syncwarp();
      if (lane == 0)
        for (int c = 0; c < 4; ++c) {
          mbar_expect_tx(my_hbar + c, GP_BOX);
          tma_load_2d(my_boxes + c * GP_BOX, &map_h, my_hbar + c, n0 + c * 32, row0);
        }
      bool good = true;
      for (int c = 0; c < GP_BN / 32; ++c, ++n_hload) {
        const int k = n_hload & 3;
        good = __all_sync(0xffffffffu, mbar_wait(my_hbar + k, (n_hload >> 2) & 1));
        if (!good) break;
        uint32_t f[32];
        unsigned char* box = my_boxes + k * GP_BOX;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 v = *gp_box_chunk(box, lane, j);
          f[4 * j + 0] = __float_as_uint(__uint_as_float(v.x) * inv);
          f[4 * j + 1] = __float_as_uint(__uint_as_float(v.y) * inv);
          f[4 * j + 2] = __float_as_uint(__uint_as_float(v.z) * inv);
          f[4 * j + 3] = __float_as_uint(__uint_as_float(v.w) * inv);
        }
        __syncwarp();                                     // every lane has read the staging tile
        if (lane == 0 && c + 4 < GP_BN / 32) {
          mbar_expect_tx(my_hbar + k, GP_BOX);
          tma_load_2d(box, &map_h, my_hbar + k, n0 + (c + 4) * 32, row0);
        }
        gp_tmem_st32(lane_taddr + buf * GP_BN + c * 32, f);
      }
      if (!good) {
        // loads that may still be in flight get the time to land before the block's shared memory goes away
        for (int i = 0; i < 1000; ++i) __nanosleep(100);
        return false;
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      fence_before();
      __syncwarp();
      if (lane == 0 && !beside) mbar_arrive_cluster(acc_empty_addr[buf]);
      return true;
    };

    if (EPI == 2) {
      if (beside) {
        if (pair < n_tiles) ok = preload(pair, 1);
      } else {
        int tile = pair;
        for (uint32_t b = 0; b < 2 && tile < n_tiles && ok; ++b, tile += n_pairs) ok = preload(tile, b);
      }
    }
    uint32_t tcount = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++tcount) {
      const int row0 = (tile % n_m) * GP_BM + (int)rank * 128 + q * 32, n0 = (tile / n_m) * GP_BN;
      const uint32_t buf = tcount & 1;
      const int row = row0 + lane;
      // the tile's bias and norm weights, once for all rows (the previous tile's readers are past their last read:
      // they have met at the barrier after it); every thread comes here, whatever its outcome so far
      if (!gp_epilogue_all<EPI_THREADS>(ok)) { ok = false; break; }
      for (int c = t; c < GP_BN; c += EPI_THREADS) {
        const int n = n0 + c;
        s_bias[c] = (a.bias && n < a.N) ? a.bias[n] : __float2bfloat16(0.0f);
        if (EPI == 2)
          s_normw[c] = n >= a.N ? 0.0f : a.norm_w_f32 ? __ldg(static_cast<const float*>(a.norm_w) + n)
                                                     : __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(a.norm_w) + n));
      }
      const float k_row = (EPI == 2 ? a.rho : 1.0f) * row_factor(row);
      const float k_bias = EPI == 2 ? a.rho : 1.0f;
      const bool plain = a.bias == nullptr && a.ss_in == nullptr && EPI != 2;      // the accumulator as it is
      // 3: the row's sines and cosines, its page, and whether the warp's rows are 32 consecutive places of one
      // page (all of this while the tile's products run)
      float rc[EPI == 3 ? 32 : 1], rs[EPI == 3 ? 32 : 1];
      int my_pos = 0, my_page = -1, pos0 = 0, page0 = -1;
      bool together = false;
      if (EPI == 3) {
        int my_seq = -1;
        if (row < a.M) { my_pos = __ldg(a.tok_pos + row); my_seq = __ldg(a.tok_seq + row); }
        const float p = (float)my_pos * a.pos_scale;
#pragma unroll
        for (int d = 0; d < 32; ++d) {
          if (a.inv_freq) rope_sincos(p, __ldg(a.inv_freq + d), a.inv_freq_lo ? __ldg(a.inv_freq_lo + d) : 0.0f, &rs[d], &rc[d]);
          else { rc[d] = 1.0f; rs[d] = 0.0f; }
        }
        if (a.write_kv && row < a.M) my_page = __ldg(a.block_table + (int64_t)my_seq * a.bt_stride + my_pos / 64);
        pos0 = __shfl_sync(0xffffffffu, my_pos, 0);
        page0 = __shfl_sync(0xffffffffu, my_page, 0);
        const int seq0 = __shfl_sync(0xffffffffu, my_seq, 0);
        together = __all_sync(0xffffffffu, row < a.M && my_seq == seq0 && my_pos == pos0 + lane && my_page >= 0) && (pos0 & 31) == 0;
      }
      // (also the barrier after which the staged bias and norm weights may be read) one outcome for all epilogue
      // threads, so that they leave the loop together
      if (!gp_epilogue_all<EPI_THREADS>(mbar_wait(acc_full + buf, (tcount >> 1) & 1))) { ok = false; break; }
      fence_after();
      const uint32_t taddr = lane_taddr + buf * GP_BN;
      float sq = 0.0f;
#pragma unroll 1
      for (int s = s_lo; s < s_hi; ++s) {                   // 64 accumulator columns at a time
        uint32_t r0[32], r1[32];
        __syncwarp();
        tmem_ld32_issue(taddr + s * 64, r0);
        tmem_ld32_issue(taddr + s * 64 + 32, r1);
        if (EPI == 0 || EPI == 3 || (EPI == 1 && (s & 1) == 0)) {
          // the store before the last one used this staging tile
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
        }
        tmem_ld_wait(r0);
        tmem_ld_wait(r1);
        float v[64];
        if (plain) {
#pragma unroll
          for (int j = 0; j < 32; ++j) { v[j] = __uint_as_float(r0[j]); v[32 + j] = __uint_as_float(r1[j]); }
        } else if (a.bias == nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) { v[j] = __uint_as_float(r0[j]) * k_row; v[32 + j] = __uint_as_float(r1[j]) * k_row; }
        } else {
#pragma unroll
          for (int j8 = 0; j8 < 8; ++j8) {
            const uint4 b8 = *reinterpret_cast<const uint4*>(s_bias + s * 64 + 8 * j8);      // eight bfloat16
            const uint32_t bw[4] = {b8.x, b8.y, b8.z, b8.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float lo = __uint_as_float(bw[e] << 16), hi = __uint_as_float(bw[e] & 0xffff0000u);
              const int j = 8 * j8 + 2 * e;
              v[j] = fmaf(__uint_as_float(j < 32 ? r0[j] : r1[j - 32]), k_row, k_bias * lo);
              v[j + 1] = fmaf(__uint_as_float(j < 32 ? r0[j + 1] : r1[j - 31]), k_row, k_bias * hi);
            }
          }
        }
        if (EPI == 2 && beside) {
          // the residual from the other accumulator
          tmem_ld32_issue(lane_taddr + GP_BN + s * 64, r0);
          tmem_ld32_issue(lane_taddr + GP_BN + s * 64 + 32, r1);
          tmem_ld_wait(r0);
          tmem_ld_wait(r1);
#pragma unroll
          for (int j = 0; j < 32; ++j) { v[j] += __uint_as_float(r0[j]); v[32 + j] += __uint_as_float(r1[j]); }
        }
        if (EPI == 0) {
          unsigned char* box = my_boxes + (n_store & 1) * GP_BOX;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *gp_box_chunk(box, lane, j) = make_uint4(gp_pack(v[8 * j], v[8 * j + 1]), gp_pack(v[8 * j + 2], v[8 * j + 3]),
                                                     gp_pack(v[8 * j + 4], v[8 * j + 5]), gp_pack(v[8 * j + 6], v[8 * j + 7]));
          fence_smem_to_tma();
          __syncwarp();
          if (lane == 0) {
            if (row0 < a.M && n0 + s * 64 < a.N) tma_store_2d(&map_y, box, n0 + s * 64, row0);
            else tma_store_skip();
          }
          ++n_store;
        } else if (EPI == 3) {
          const int col = n0 + s * 64, head = col >> 6;
          if (col < a.N) {                                  // (the same for the whole warp)
            // as the plain epilogue would store it, then rotated: pairs d, d + 32
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
            if (head < a.nh + a.nkv) {
#pragma unroll
              for (int d = 0; d < 32; ++d) {
                const float x0 = v[d], x1 = v[d + 32];
                v[d] = x0 * rc[d] - x1 * rs[d];
                v[d + 32] = x1 * rc[d] + x0 * rs[d];
              }
            }
            uint4 o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              o[j] = make_uint4(gp_pack(v[8 * j], v[8 * j + 1]), gp_pack(v[8 * j + 2], v[8 * j + 3]),
                                gp_pack(v[8 * j + 4], v[8 * j + 5]), gp_pack(v[8 * j + 6], v[8 * j + 7]));
            const bool is_q = head < a.nh;
            const bool is_k = !is_q && head < a.nh + a.nkv;
            const int g = is_k ? head - a.nh : head - a.nh - a.nkv;
            if (is_q || (a.write_kv && together)) {
              unsigned char* box = my_boxes + (n_store & 1) * GP_BOX;
#pragma unroll
              for (int j = 0; j < 8; ++j) *gp_box_chunk(box, lane, j) = o[j];
              fence_smem_to_tma();
              __syncwarp();
              if (lane == 0) {
                if (is_q) {
                  if (row0 < a.M) tma_store_2d(&map_y, box, col, row0); else tma_store_skip();
                } else {
                  tma_store_2d(is_k ? &map_k : &map_v, box, 0, (page0 * a.nkv + g) * 64 + (pos0 & 63));
                }
              }
              ++n_store;
            } else if (a.write_kv && row < a.M && my_page >= 0) {
              uint4* dst = reinterpret_cast<uint4*>((is_k ? a.k_pool : a.v_pool) +
                                                    (((int64_t)my_page * a.nkv + g) * 64 + (my_pos & 63)) * 64);
#pragma unroll
              for (int j = 0; j < 8; ++j) dst[j] = o[j];
            }
          }
        } else if (EPI == 1) {
          // four groups of (8 gate, 8 up) -> 32 outputs: half a staging tile
          unsigned char* box = my_boxes + (n_store & 1) * GP_BOX;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float gate = v[g * 16 + j], up = v[g * 16 + 8 + j];
              o[j] = __fdividef(gate, 1.0f + __expf(-gate)) * up;
            }
            *gp_box_chunk(box, lane, (s & 1) * 4 + g) = make_uint4(gp_pack(o[0], o[1]), gp_pack(o[2], o[3]), gp_pack(o[4], o[5]), gp_pack(o[6], o[7]));
          }
          if (s & 1) {
            fence_smem_to_tma();
            __syncwarp();
            if (lane == 0) {
              if (row0 < a.M && n0 + (s >> 1) * 128 < a.N) tma_store_2d(&map_y, box, (n0 >> 1) + (s >> 1) * 64, row0);
              else tma_store_skip();
            }
            ++n_store;
          }
        } else {
          // v is the new h (columns beyond N: zero in h, in the products and in the staged bias).  Per step two
          // float32 tiles of it and one bfloat16 tile of x_raw go out, in this order; a staging tile is written
          // again a step later (x_raw's: two steps), when all but the two newest stores have read theirs.
          unsigned char* xbox = my_boxes + (2 + (s & 1)) * GP_BOX;
#pragma unroll
          for (int j = 0; j < 64; ++j) sq = fmaf(v[j], v[j], sq);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            unsigned char* hbox = my_boxes + half * GP_BOX;
            if (lane == 0) tma_store_wait_read<2>();
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float* f = v + 32 * half + 4 * j;
              *gp_box_chunk(hbox, lane, j) = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float* f = v + 32 * half + 8 * j;
              const float* wn = s_normw + s * 64 + 32 * half + 8 * j;
              *gp_box_chunk(xbox, lane, 4 * half + j) = make_uint4(gp_pack(f[0] * wn[0], f[1] * wn[1]), gp_pack(f[2] * wn[2], f[3] * wn[3]),
                                                                   gp_pack(f[4] * wn[4], f[5] * wn[5]), gp_pack(f[6] * wn[6], f[7] * wn[7]));
            }
            fence_smem_to_tma();
            __syncwarp();
            if (lane == 0 && row0 < a.M) {
              if (n0 + s * 64 + 32 * half < a.N) tma_store_2d(&map_h, hbox, n0 + s * 64 + 32 * half, row0);
              else tma_store_skip();
              if (half == 1) {
                if (n0 + s * 64 < a.N) tma_store_2d(&map_y, xbox, n0 + s * 64, row0);
                else tma_store_skip();
              }
            }
          }
        }
      }
      if (EPI == 2) {
        if (row < a.M) a.ss_out[(int64_t)row * n_n + tile / n_m] = sq;
        // the accumulator is free: the tile after next of this pair goes into it (or nobody waits for it)
        const int next = tile + 2 * n_pairs;
        fence_before();
        if (next < n_tiles) ok = preload(next, buf);
      } else {
        fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_addr[buf]);
      }
    }
    if (!ok && lane == 0) atomicExch(&g_gp_error, 3);
  }

  fence_before();
  cluster_arrive_all();
  // (meanwhile) the stores have read their staging tiles; the kernel's end covers the rest of their way
  if (warp >= 2 && lane == 0) tma_store_wait_read<0>();
  __syncwarp();
  cluster_wait_all();                          // nobody reads the partner's shared or tensor memory after this
  fence_after();
  if (warp == 1) tmem_free_pair<512>(tmem_base);
}

template <int EPI> static const void* gp_kernel() { return reinterpret_cast<const void*>(&gemm_pair_kernel<EPI>); }

// attr: room for two attributes.
static void gp_launch_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int blocks, int epi, cudaStream_t stream) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(blocks);
  cfg->blockDim = dim3(gp_threads(epi));
  cfg->dynamicSmemBytes = gp_smem(epi);
  cfg->stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg->attrs = attr;
  cfg->numAttrs = pdl_enabled() ? 2 : 1;
}

// Pairs that the GPU runs at once (a pair needs two SMs of one cluster-capable group).
static int gp_max_pairs(int epi) {
  static int pairs[4] = {0, 0, 0, 0};
  if (pairs[epi]) return pairs[epi];
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int n = sms / 2;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  gp_launch_config(&cfg, attr, sms & ~1, epi, nullptr);
  cfg.numAttrs = 1;
  int clusters = 0;
  const void* fn = epi == 0 ? gp_kernel<0>() : epi == 1 ? gp_kernel<1>() : epi == 2 ? gp_kernel<2>() : gp_kernel<3>();
  if (cudaOccupancyMaxActiveClusters(&clusters, fn, &cfg) == cudaSuccess && clusters > 0 && clusters < n) n = clusters;
  cudaGetLastError();
  pairs[epi] = n > 0 ? n : 1;
  return pairs[epi];
}

}  // namespace exl3

using namespace exl3;

// 0 when no kernel has given up on a wait since the last call; else 1 (producer), 2 (MMA), 3 (epilogue).
extern "C" int exl3_gemm_pair_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_gp_error, sizeof(int));
  if (v) { int z = 0; cudaMemcpyToSymbol(g_gp_error, &z, sizeof(int)); }
  return v;
}

// The common part of the two entry points: `a` and `pools` carry what the epilogue needs beyond y.
static int gp_run(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int epilogue,
                  const float* ss_in, int ss_blocks, float eps, float width, float* h, PairArgs a, int64_t pool_rows,
                  cudaStream_t stream) {
  if (!aligned16(x) || !aligned16(w) || (y && !aligned16(y))) { set_error("gemm_pair: x, w and y must be 16-byte aligned"); return ERR_ALIGNMENT; }
  if (ss_in && (ss_blocks < 1 || !(width > 0.0f))) { set_error("gemm_pair: the norm's pieces need blocks >= 1 and a width"); return ERR_BAD_ARGUMENT; }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gp_smem(0));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gp_smem(1));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_pair_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gp_smem(2));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_pair_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gp_smem(3));
    if (e != cudaSuccess) { set_error("gemm_pair: cannot get %u bytes of shared memory: %s", gp_smem(2), cudaGetErrorString(e)); return (int)e; }
    configured = true;
  }
  CUtensorMap map_x, map_w, map_y, map_h, map_k, map_v;
  int rc = make_map_k64(&map_x, x, M, K, 128, "gemm_pair");
  if (rc) return rc;
  rc = make_map_k64(&map_w, w, N, K, 128, "gemm_pair");
  if (rc) return rc;
  rc = make_map_128b(&map_y, y, M, epilogue == 1 ? N / 2 : N, 2, 32, "gemm_pair");
  if (rc) return rc;
  map_h = map_k = map_v = map_y;
  if (epilogue == 2) {
    rc = make_map_128b(&map_h, h, M, N, 4, 32, "gemm_pair");
    if (rc) return rc;
  }
  if (epilogue == 3 && a.write_kv) {
    rc = make_map_128b(&map_k, a.k_pool, pool_rows, 64, 2, 32, "gemm_pair");
    if (rc) return rc;
    rc = make_map_128b(&map_v, a.v_pool, pool_rows, 64, 2, 32, "gemm_pair");
    if (rc) return rc;
  }
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.M = M; a.N = N; a.K = K;
  a.ss_in = ss_in; a.ss_blocks = ss_blocks; a.eps = eps; a.width = width;
  const int tiles = ceil_div(M, GP_BM) * ceil_div(N, GP_BN);
  const int max_pairs = gp_max_pairs(epilogue);
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  gp_launch_config(&cfg, attr, 2 * pairs, epilogue, stream);
  cudaError_t e;
  if (epilogue == 0) e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<0>, map_x, map_w, map_y, map_h, map_k, map_v, a);
  else if (epilogue == 1) e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<1>, map_x, map_w, map_y, map_h, map_k, map_v, a);
  else if (epilogue == 2) e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<2>, map_x, map_w, map_y, map_h, map_k, map_v, a);
  else e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<3>, map_x, map_w, map_y, map_h, map_k, map_v, a);
  if (e != cudaSuccess) { set_error("gemm_pair: launch failed: %s", cudaGetErrorString(e)); return (int)e; }
  return launch_status("gemm_pair");
}

extern "C" int exl3_gemm_pair(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                              int epilogue, const float* ss_in, int ss_blocks, float eps, float width, float* h,
                              float rho, const void* norm_w, int norm_w_dtype, void* x_raw, float* ss_out,
                              cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || N < 0 || K < 8 || K % 8 != 0 || N % 8 != 0 || epilogue < 0 || epilogue > 2 || (epilogue == 1 && N % 16 != 0)) {
    set_error("gemm_pair: needs K and N multiples of 8 (N of 16 with the gated epilogue) and epilogue 0, 1 or 2, got M=%d N=%d K=%d epilogue %d",
              M, N, K, epilogue);
    return ERR_BAD_ARGUMENT;
  }
  PairArgs a = {};
  if (epilogue == 2) {
    if (!h || !norm_w || !x_raw || !ss_out || !aligned16(h) || !aligned16(x_raw) ||
        (norm_w_dtype != DT_F32 && norm_w_dtype != DT_BF16) || !(rho != 0.0f)) {
      set_error("gemm_pair: the residual epilogue needs h, norm_w (float32 or bfloat16), x_raw and ss_out, 16-byte aligned, and a scale that is not zero");
      return ERR_BAD_ARGUMENT;
    }
    a.rho = rho; a.norm_w = norm_w; a.norm_w_f32 = norm_w_dtype == DT_F32 ? 1 : 0;
    a.ss_out = ss_out;
  }
  return gp_run(x, w, bias, epilogue == 2 ? x_raw : y, M, N, K, epilogue, ss_in, ss_blocks, eps, width, h, a, 0, stream);
}

// The q/k/v projection of nh query and nkv key/value heads of 64 with the rotary encoding (rot = 64, or 0 for
// none) and the cache write in its epilogue: y is [M, (nh + 2 nkv) * 64], of which the queries' columns are written;
// keys and values go to the pools [pool_rows / (nkv * 64) pages, nkv, 64, 64] when write_kv is set.
extern "C" int exl3_gemm_pair_rope(const void* x, const void* w, const void* bias, void* y, int M, int K,
                                   const float* ss_in, int ss_blocks, float eps, float width, const int* tok_pos,
                                   const int* tok_seq, const int* block_table, int bt_stride, const float* inv_freq,
                                   const float* inv_freq_lo, int rot, float pos_scale, int nh, int nkv, int hd,
                                   int page, void* k_pool, void* v_pool, int64_t pool_rows, int write_kv,
                                   cudaStream_t stream) {
  if (M == 0) return 0;
  if (M < 0 || K < 8 || K % 8 != 0 || nh < 1 || nkv < 1 || hd != 64 || page != 64 || (rot != 0 && rot != 64) ||
      (rot != 0 && !inv_freq) || !tok_pos || !tok_seq || (write_kv && (!block_table || !k_pool || !v_pool || pool_rows < 64))) {
    set_error("gemm_pair_rope: needs heads of 64 rotated as a whole or not at all, pages of 64, K a multiple of 8, positions and "
              "(to write the cache) a block table and pools; got M=%d K=%d heads=%d kv_heads=%d head_dim=%d page=%d rot=%d",
              M, K, nh, nkv, hd, page, rot);
    return ERR_BAD_ARGUMENT;
  }
  if (write_kv && (!aligned16(k_pool) || !aligned16(v_pool))) { set_error("gemm_pair_rope: the pools must be 16-byte aligned"); return ERR_ALIGNMENT; }
  PairArgs a = {};
  a.tok_pos = tok_pos; a.tok_seq = tok_seq; a.block_table = block_table; a.bt_stride = bt_stride;
  a.inv_freq = rot ? inv_freq : nullptr; a.inv_freq_lo = rot ? inv_freq_lo : nullptr; a.pos_scale = pos_scale;
  a.nh = nh; a.nkv = nkv; a.write_kv = write_kv ? 1 : 0;
  a.k_pool = static_cast<__nv_bfloat16*>(k_pool); a.v_pool = static_cast<__nv_bfloat16*>(v_pool);
  return gp_run(x, w, bias, y, M, (nh + 2 * nkv) * 64, K, 3, ss_in, ss_blocks, eps, width, nullptr, a, pool_rows, stream);
}

// Tiles of 256 columns per row in ss_out of the residual epilogue.
extern "C" int exl3_gemm_pair_ss_blocks(int N) { return ceil_div(N, GP_BN); }
