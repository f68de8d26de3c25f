// Prefill-shaped projection on the 5th-generation tensor cores:
//   y[M,N] = x[M,K] . w[N,K]^T (+ bias), bfloat16 operands, float32 accumulation
// with an optional gated epilogue (the feed-forward's silu(gate) * up, for a
// weight whose rows are 8 gate rows, the 8 up rows of the same features, ...),
// so the gate/up product never goes to memory.  In the reference these are
// library matmuls followed by separate sigmoid and multiply ops
// (src/model.cpp:583-586).
//
// Structure (one persistent block per SM, 6 warps):
//   warp 0    TMA producer: cp.async.bulk.tensor copies 128x64 tiles of x and
//             256x64 tiles of w into a 4-stage ring of 128B-swizzled shared memory
//   warp 1    MMA issuer: one thread issues tcgen05.mma (M128 N256 K16, operands
//             from shared-memory descriptors, accumulator in tensor memory);
//             tcgen05.commit releases ring stages and hands accumulators over
//   warps 2-5 epilogue: tcgen05.ld the accumulator (each warp its 32 lanes),
//             bias / activation / bfloat16, 16-byte stores
// Two accumulator buffers (2 x 256 of the 512 TMEM columns) let the epilogue of
// one tile overlap the main loop of the next.  Tiles go round-robin over the
// blocks, M fastest, so blocks that run together share a tile of w in L2.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the kernel
// records an error code, leaves its loops, waits (bounded) for copies it has in
// flight, frees its tensor memory and returns; exl3_gemm_tc_status() reads the
// code.  No cluster, no multicast.
#include "api.h"
#include "common.cuh"

#include <cuda.h>

#include <mutex>
#include <unordered_map>

namespace exl3 {

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 64, TC_STAGES = 4, TC_UMMA_K = 16;
constexpr int TC_THREADS = 192;
constexpr int TC_TMEM_COLS = 512;
constexpr uint32_t TC_STAGE_A = TC_BM * TC_BK * 2, TC_STAGE_B = TC_BN * TC_BK * 2;
constexpr uint32_t TC_SMEM = TC_STAGES * (TC_STAGE_A + TC_STAGE_B) + 1024 /* alignment */ + 256 /* barriers */;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;   // polls of a few tens of nanoseconds each: well under a second

static __device__ int g_tc_error = 0;

__device__ inline uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ inline void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ inline void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ inline void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ inline bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = TC_WAIT_LIMIT) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
    if (i > 64) __nanosleep(32);
  }
  return false;
}
__device__ inline void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ inline void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand tile in 128B-swizzled shared memory: rows of 128 bytes, groups
// of 8 rows 1024 bytes apart (descriptor fields as in CUTLASS's
// cute/arch/mma_sm100_desc.hpp: start >> 4, leading offset 1, stride offset
// 1024 >> 4, version 1, layout SWIZZLE_128B = 2).
__device__ inline uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3fff) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: D float32, A and B bfloat16, both K-major, N = 256, M = 128.
constexpr uint32_t TC_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((TC_BN >> 3) << 17) | ((TC_BM >> 4) << 24);

__device__ inline void umma(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(da), "l"(db), "r"(TC_IDESC), "r"(accumulate), "r"(0u) : "memory");
}
__device__ inline void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// epi 0: y[M,N] bf16.  epi 1: y[M,N/2] = silu(gate) * up, rows of w interleaved in eights.
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
               int epi) {
  extern __shared__ unsigned char tc_smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = base;
  unsigned char* sB = base + TC_STAGES * TC_STAGE_A;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + TC_STAGES * (TC_STAGE_A + TC_STAGE_B));
  uint64_t* full = bars;                       // [STAGES] copies landed
  uint64_t* empty = bars + TC_STAGES;          // [STAGES] MMAs that read the stage are done
  uint64_t* acc_full = bars + 2 * TC_STAGES;   // [2] accumulator complete
  uint64_t* acc_empty = acc_full + 2;          // [2] accumulator read out
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TC_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_m = (M + TC_BM - 1) / TC_BM, n_n = (N + TC_BN - 1) / TC_BN;
  const int n_tiles = n_m * n_n, kblocks = (K + TC_BK - 1) / TC_BK;
  bool ok = true;

  if (warp == 0) {
    // ---- producer -----------------------------------------------------------
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile % n_m) * TC_BM, n0 = (tile / n_m) * TC_BN;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % TC_STAGES;
        if (!mbar_wait(empty + s, ((it / TC_STAGES) & 1) ^ 1)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(full + s, TC_STAGE_A + TC_STAGE_B);
          tma_load_2d(sA + s * TC_STAGE_A, &map_x, full + s, kb * TC_BK, m0);
          tma_load_2d(sB + s * TC_STAGE_B, &map_w, full + s, kb * TC_BK, n0);
        }
        __syncwarp();
      }
    }
    if (!ok && lane == 0) atomicExch(&g_tc_error, 1);
    // copies still in flight must land before the block's shared memory goes away
    if (!ok) {
      for (uint32_t back = 1; back <= (uint32_t)TC_STAGES && back <= it; ++back) {
        const uint32_t j = it - back;
        mbar_wait(full + (j % TC_STAGES), (j / TC_STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -----------------------------------------------------------
    uint32_t it = 0, tcount = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tcount) {
      const uint32_t buf = tcount & 1;
      if (!mbar_wait(acc_empty + buf, ((tcount >> 1) & 1) ^ 1)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * TC_BN;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % TC_STAGES;
        if (!mbar_wait(full + s, (it / TC_STAGES) & 1)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint64_t da = umma_desc(smem_u32(sA + s * TC_STAGE_A));
          const uint64_t db = umma_desc(smem_u32(sB + s * TC_STAGE_B));
#pragma unroll
          for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)     // 32 bytes further along K: start address + 2
            umma(d_tmem, da + 2 * k, db + 2 * k, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty + s);
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) umma_commit(acc_full + buf);
      __syncwarp();
    }
    if (!ok && lane == 0) atomicExch(&g_tc_error, 2);
  } else {
    // ---- epilogue ---------------------------------------------------------------
    const int q = warp & 3;                               // the 32 TMEM lanes this warp may read
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tcount) {
      const int m0 = (tile % n_m) * TC_BM, n0 = (tile / n_m) * TC_BN;
      const uint32_t buf = tcount & 1;
      if (!mbar_wait(acc_full + buf, (tcount >> 1) & 1)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * TC_BN;
#pragma unroll 1
      for (int c = 0; c < TC_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        const int col = n0 + c * 32;
        if (row >= M || col >= N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j) if (col + j < N) v[j] += __bfloat162float(bias[col + j]);
        }
        if (epi == 1) {
          // two groups of (8 gate, 8 up) -> 16 outputs
          float o[16];
#pragma unroll
          for (int g2 = 0; g2 < 2; ++g2)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float g = v[g2 * 16 + j], u = v[g2 * 16 + 8 + j];
              o[g2 * 8 + j] = __fdividef(g, 1.0f + __expf(-g)) * u;
            }
          __nv_bfloat16* dst = y + (int64_t)row * (N >> 1) + (col >> 1);
          const float o0[8] = {o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]};
          store_vec(dst, o0);
          if (col + 16 < N) {
            const float o1[8] = {o[8], o[9], o[10], o[11], o[12], o[13], o[14], o[15]};
            store_vec(dst + 8, o1);
          }
        } else {
          __nv_bfloat16* dst = y + (int64_t)row * N + col;
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            if (col + p * 8 + 8 <= N) {
              const float o8[8] = {v[p * 8], v[p * 8 + 1], v[p * 8 + 2], v[p * 8 + 3],
                                   v[p * 8 + 4], v[p * 8 + 5], v[p * 8 + 6], v[p * 8 + 7]};
              store_vec(dst + p * 8, o8);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + buf);
    }
    if (!ok && lane == 0) atomicExch(&g_tc_error, 3);
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
}

// A wait that nothing will ever satisfy, with a short limit: shows that a kernel
// of this file gives up, records its code (9) and returns, leaving the context usable.
__global__ void wait_selftest_kernel() {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (!mbar_wait(&bar, 0, 1u << 14) && threadIdx.x == 0) atomicExch(&g_tc_error, 9);
}

// ---- host side --------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// A [rows, K] bfloat16 row-major matrix, boxes of box_rows x 64 columns, 128B swizzle, zero fill outside.
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("gemm_tc: the driver has no cuTensorMapEncodeTiled"); return ERR_UNSUPPORTED; }
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("gemm_tc: cuTensorMapEncodeTiled failed with %d", (int)r); return ERR_BAD_ARGUMENT; }
  return 0;
}

static int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

}  // namespace exl3

using namespace exl3;

// 0 when no kernel has given up on a wait since the last call; else 1 (producer), 2 (MMA), 3 (epilogue).
extern "C" int exl3_gemm_tc_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int));
  if (v) { int z = 0; cudaMemcpyToSymbol(g_tc_error, &z, sizeof(int)); }
  return v;
}

extern "C" int exl3_gemm_tc_wait_selftest(cudaStream_t stream) {
  wait_selftest_kernel<<<1, 32, 0, stream>>>();
  return launch_status("gemm_tc_wait_selftest");
}

extern "C" int exl3_gemm_tc(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                            int epilogue, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || N < 0 || K < 8 || K % 8 != 0 || N % 8 != 0 || (epilogue != 0 && (epilogue != 1 || N % 16 != 0))) {
    set_error("gemm_tc: needs K and N multiples of 8 (N of 16 with the gated epilogue), got M=%d N=%d K=%d", M, N, K);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(x) || !aligned16(w) || !aligned16(y)) { set_error("gemm_tc: x, w and y must be 16-byte aligned"); return ERR_ALIGNMENT; }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
    if (e != cudaSuccess) { set_error("gemm_tc: cannot get %u bytes of shared memory: %s", TC_SMEM, cudaGetErrorString(e)); return (int)e; }
    configured = true;
  }
  CUtensorMap map_x, map_w;
  int rc = make_map(&map_x, x, M, K, TC_BM);
  if (rc) return rc;
  rc = make_map(&map_w, w, N, K, TC_BN);
  if (rc) return rc;
  const int tiles = ceil_div(M, TC_BM) * ceil_div(N, TC_BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_tc_kernel<<<grid, TC_THREADS, TC_SMEM, stream>>>(map_x, map_w, static_cast<__nv_bfloat16*>(y),
                                                         static_cast<const __nv_bfloat16*>(bias), M, N, K, epilogue);
  return launch_status("gemm_tc");
}
