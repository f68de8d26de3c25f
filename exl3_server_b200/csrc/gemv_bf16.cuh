// Decode-shaped projection: y[M,N] = x[M,K] . w[N,K]^T (+ bias) for M <= 16
// rows of x, bfloat16 operands, float32 accumulation.
//
// The weight matrix is read exactly once, in 16-byte pieces that go as they
// are into the A fragments of mma.m16n8k16 (weights are the 16-row operand,
// the batch is the 8-column one).  No change of layout is needed because the
// order of the K index inside a 32-wide block is free: a thread's 8
// consecutive weights and its 8 consecutive activations are assigned to the
// same logical k slots of two mma instructions.  Shared memory only holds the
// pieces on their way (a ring per thread, filled by cp.async).
//
// A block owns 16 output features; its warps take 32-wide K blocks in turn and
// their partial tiles are summed in warp order, so a result depends on K, N
// and the warp count only, never on M or the batch's other rows.
#pragma once
#include "api.h"
#include "common.cuh"

#include <algorithm>

namespace exl3 {

__device__ inline uint4 ldg_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

__device__ inline void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int GEMV_MAX_WARPS = 16;

// 16 bytes global -> shared without passing through registers; src_bytes 0 writes zeros.
__device__ inline void cp_async16_zfill(void* smem, const void* gmem, int src_bytes) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ inline void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ inline void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A thread streams its own pieces of the weights (rows gid and gid + 8 of the
// block's 16, the 16 bytes at tig * 8 of each 32-wide K block its warp owns)
// through a ring of GEMV_STAGES (4 or 6) slots in shared memory with cp.async.  Only the
// thread that copied a slot reads it, so the ring needs no block barrier, costs
// no registers, and keeps (GEMV_STAGES - 1) * 32 bytes of weights per thread in
// flight.  Its pieces of the activations travel in the same ring.
//
// The norm between two projections, without a kernel of its own (GemvNorm):
//   h += y * rho;   r = h * rsqrt(mean(h^2) + eps) * norm_w;   y2 = r . w2^T
// is done in pieces.  The projection that produces y (EPI 2) keeps no y: each of its blocks adds its 16 features
// to the float32 residual h, writes them times the norm weight as bfloat16 (x_raw) and writes the sums of their
// squares per batch row (ss_part[16][blocks]).  The projection that consumes r (SCALE) reads x_raw as its input,
// adds the blocks' sums in an order that depends on its thread count only, and multiplies its results by
// rsqrt(sum / width + eps) before bias and gating: a factor per batch row commutes with the product.  Statistics and the residual stay float32.
struct GemvNorm {
  // EPI 2, the producing side
  float* h;                      // [M, N] residual, updated in place
  const void* norm_w;            // [N] weight of the norm that follows
  __nv_bfloat16* x_raw;          // [M, N] out: h * norm_w
  float* ss_out;                 // [16, blocks] out: sums of squares of the block's features, per batch row
  float rho;
  int norm_w_f32;
  // SCALE, the consuming side
  const float* ss_in;            // [16, ss_blocks] from the producer
  int ss_blocks;
  float eps, width;
};

// EPI 0: y[m, n] = acc (+ bias).  EPI 1 (gated feed-forward): the 16 rows of a
// block are 8 gate rows followed by the 8 up rows of the same features;
// y[m, block * 8 + r] = silu(gate_r) * up_r, so N / 2 features come out.
template <int NT, typename TO, int EPI, int GEMV_STAGES, bool SCALE = false>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32)
gemv_bf16_kernel(const __nv_bfloat16* x, const __nv_bfloat16* __restrict__ w,
                 const __nv_bfloat16* __restrict__ bias, TO* __restrict__ y, int M, int N, int K, GemvNorm nrm) {
  __shared__ float s_inv[16];                           // SCALE: rsqrt(mean square + eps) of each batch row
  extern __shared__ uint4 ring[];                     // [GEMV_STAGES][2 + NT][blockDim.x]: weights a, b, then x
  pdl_trigger();
  const int tid = threadIdx.x, nthreads = blockDim.x;
  // partial tiles of the warps, [warps][16][8 NT + 1]: in the ring's place, once every thread is done with the ring
  // (kept apart they cost the q/k/v projection its third block per SM: 3 x 78 KB do not fit, and its 432 blocks
  // then run as one and a half waves)
  float (*part)[16][8 * NT + 1] = reinterpret_cast<float (*)[16][8 * NT + 1]>(ring);
  const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int r0 = blockIdx.x * 16;
  const int row_a = r0 + gid, row_b = r0 + gid + 8;
  const bool ok_a = row_a < N, ok_b = row_b < N;
  const __nv_bfloat16* wa = w + (int64_t)(ok_a ? row_a : 0) * K;
  const __nv_bfloat16* wb = w + (int64_t)(ok_b ? row_b : 0) * K;
  float c[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) c[t][i] = 0.0f;
  const int nblocks = (K + 31) / 32;
  const int n_my = warp < nblocks ? (nblocks - warp + nwarps - 1) / nwarps : 0;   // K blocks of this warp
  constexpr int SLOTS = 2 + NT;
  auto issue_w = [&](int i) {
    const int k = (warp + i * nwarps) * 32 + tig * 8;
    const bool in = k < K;                            // K % 8 == 0: a piece is inside or outside
    const int st = i % GEMV_STAGES;
    cp_async16_zfill(&ring[(st * SLOTS + 0) * nthreads + tid], wa + (in ? k : 0), (in && ok_a) ? 16 : 0);
    cp_async16_zfill(&ring[(st * SLOTS + 1) * nthreads + tid], wb + (in ? k : 0), (in && ok_b) ? 16 : 0);
  };
  // the activations take the same road (cp.async.cg reads through L2, which is what data
  // written by the previous kernel needs), so no load latency is exposed in the loop
  auto issue_x = [&](int i) {
    const int k = (warp + i * nwarps) * 32 + tig * 8;
    const bool in = k < K;
    const int st = i % GEMV_STAGES;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int m = t * 8 + gid;
      const bool okx = in && m < M;
      cp_async16_zfill(&ring[(st * SLOTS + 2 + t) * nthreads + tid], x + (okx ? (int64_t)m * K + k : 0), okx ? 16 : 0);
    }
  };
  // weights first: they do not depend on the kernel before this one
#pragma unroll
  for (int i = 0; i < GEMV_STAGES - 1; ++i) {
    if (i < n_my) issue_w(i);
    cp_async_commit_group();
  }
  pdl_wait();
#pragma unroll
  for (int i = 0; i < GEMV_STAGES - 1; ++i) {
    if (i < n_my) issue_x(i);
    cp_async_commit_group();
  }
  // EPI 2: the epilogue's own operands (a residual value and a norm weight per thread, when the block has at
  // least 16 * 8 * NT threads) are asked for here too
  float h_pre = 0.0f, wn_pre = 0.0f;
  if constexpr (EPI == 2) {
    const int m = tid >> 4, n = r0 + (tid & 15);
    if (tid < 16 * 8 * NT && m < M && n < N) {
      h_pre = __ldcg(nrm.h + (int64_t)m * N + n);
      wn_pre = nrm.norm_w_f32 ? __ldg(static_cast<const float*>(nrm.norm_w) + n)
                              : __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(nrm.norm_w) + n));
    }
  }
  // SCALE: the producer's sums of squares [16][ss_blocks].  Warp w adds up batch rows w, w + warps, ...: its lanes
  // take a row's values side by side.  The loads are asked for here, together with the activations, and added
  // up after the loop (an order that depends on the number of blocks only).
  constexpr int SS_ROWS = 4, SS_AHEAD = 8;               // rows per warp and values per lane asked for ahead
  float ss_v[SS_ROWS][SS_AHEAD];
  if constexpr (SCALE) {
#pragma unroll
    for (int rr = 0; rr < SS_ROWS; ++rr) {
      const int m = warp + rr * nwarps;
#pragma unroll
      for (int j = 0; j < SS_AHEAD; ++j) {
        const int p = lane + 32 * j;
        ss_v[rr][j] = (m < M && p < nrm.ss_blocks) ? __ldcg(nrm.ss_in + (int64_t)m * nrm.ss_blocks + p) : 0.0f;
      }
    }
  }
  // Groups complete in order: W0..W(S-2), X0..X(S-2), then one group per iteration.  Block i
  // needs the group at index S-1+i; at iteration i, 2(S-1)+i groups exist, so S-2 may pend.
  for (int i = 0; i < n_my; ++i) {
    cp_async_wait_group<GEMV_STAGES - 2>();
    const int st = i % GEMV_STAGES;
    const uint4 a = ring[(st * SLOTS + 0) * nthreads + tid];
    const uint4 b = ring[(st * SLOTS + 1) * nthreads + tid];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const uint4 xv = ring[(st * SLOTS + 2 + t) * nthreads + tid];
      mma_bf16(c[t], a.x, b.x, a.y, b.y, xv.x, xv.y);
      mma_bf16(c[t], a.z, b.z, a.w, b.w, xv.z, xv.w);
    }
    // the slot read above is refilled only now, after its values were used
    if (i + GEMV_STAGES - 1 < n_my) { issue_w(i + GEMV_STAGES - 1); issue_x(i + GEMV_STAGES - 1); }
    cp_async_commit_group();
  }
  cp_async_wait_group<0>();
  __syncthreads();                                     // the ring is free: the partial tiles take its place
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    part[warp][gid][t * 8 + tig * 2] = c[t][0];
    part[warp][gid][t * 8 + tig * 2 + 1] = c[t][1];
    part[warp][gid + 8][t * 8 + tig * 2] = c[t][2];
    part[warp][gid + 8][t * 8 + tig * 2 + 1] = c[t][3];
  }
  if constexpr (SCALE) {
    for (int rr = 0; warp + rr * nwarps < M; ++rr) {
      const int m = warp + rr * nwarps;
      float ss = 0.0f;
      if (rr < SS_ROWS) {
#pragma unroll
        for (int q = 0; q < SS_ROWS; ++q) {
          if (q == rr) {
#pragma unroll
            for (int j = 0; j < SS_AHEAD; ++j) ss += ss_v[q][j];
          }
        }
        for (int p = lane + 32 * SS_AHEAD; p < nrm.ss_blocks; p += 32) ss += __ldcg(nrm.ss_in + (int64_t)m * nrm.ss_blocks + p);
      } else {
        for (int p = lane; p < nrm.ss_blocks; p += 32) ss += __ldcg(nrm.ss_in + (int64_t)m * nrm.ss_blocks + p);
      }
      ss = warp_sum(ss);
      if (lane == 0) s_inv[m] = 1.0f / sqrtf(ss / nrm.width + nrm.eps);
    }
  }
  __syncthreads();
  if (EPI == 0) {
    for (int idx = threadIdx.x; idx < 16 * 8 * NT; idx += blockDim.x) {
      const int m = idx >> 4, r = idx & 15;           // consecutive threads: consecutive features
      const int n = r0 + r;
      if (m >= M || n >= N) continue;
      float s = 0.0f;
      for (int wi = 0; wi < nwarps; ++wi) s += part[wi][r][m];
      if (SCALE) s *= s_inv[m];
      if (bias) s += __bfloat162float(bias[n]);
      Elem<TO>::store(y + (int64_t)m * N + n, s);
    }
  } else if (EPI == 1) {
    const int n_out = N >> 1;
    for (int idx = threadIdx.x; idx < 8 * 8 * NT; idx += blockDim.x) {
      const int m = idx >> 3, r = idx & 7;
      const int f = blockIdx.x * 8 + r;
      if (m >= M || f >= n_out) continue;
      float g = 0.0f, u = 0.0f;
      for (int wi = 0; wi < nwarps; ++wi) { g += part[wi][r][m]; u += part[wi][r + 8][m]; }
      if (SCALE) { g *= s_inv[m]; u *= s_inv[m]; }
      if (bias) { g += __bfloat162float(bias[r0 + r]); u += __bfloat162float(bias[r0 + r + 8]); }
      Elem<TO>::store(y + (int64_t)m * n_out + f, g / (1.0f + expf(-g)) * u);
    }
  } else {
    // EPI 2: into the residual.  Whole warps take part (the limits are multiples of 32); the 16 lanes of a
    // batch row add their squares.
    for (int idx = threadIdx.x; idx < 16 * 8 * NT; idx += blockDim.x) {
      const int m = idx >> 4, r = idx & 15;
      const int n = r0 + r;
      float sq = 0.0f;
      if (m < M && n < N) {
        float s = 0.0f;
        for (int wi = 0; wi < nwarps; ++wi) s += part[wi][r][m];
        if (SCALE) s *= s_inv[m];
        if (bias) s += __bfloat162float(bias[n]);
        // the output is rounded to bfloat16 as it would be on its way through memory
        const bool first = idx == (int)threadIdx.x;     // the first pass uses what was asked for before the loop
        const float h_old = first ? h_pre : __ldcg(nrm.h + (int64_t)m * N + n);
        const float hv = h_old + __bfloat162float(__float2bfloat16_rn(s)) * nrm.rho;
        nrm.h[(int64_t)m * N + n] = hv;
        const float wn = first ? wn_pre
                       : nrm.norm_w_f32 ? static_cast<const float*>(nrm.norm_w)[n]
                                        : __bfloat162float(static_cast<const __nv_bfloat16*>(nrm.norm_w)[n]);
        nrm.x_raw[(int64_t)m * N + n] = __float2bfloat16_rn(hv * wn);
        sq = hv * hv;
      }
      sq += __shfl_xor_sync(0xffffffffu, sq, 8);
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      if (r == 0) nrm.ss_out[(int64_t)m * gridDim.x + blockIdx.x] = sq;     // zero for rows beyond M
    }
    if (NT == 1 && threadIdx.x >= 8 && threadIdx.x < 16) nrm.ss_out[(int64_t)threadIdx.x * gridDim.x + blockIdx.x] = 0.0f;
  }
}

static size_t gemv_smem(int nt, int stages, int warps) {
  return std::max((size_t)stages * (2 + nt) * warps * 32 * sizeof(uint4), (size_t)warps * 16 * (8 * nt + 1) * sizeof(float));
}

template <int NT, typename TO, int EPI, int STAGES, bool SCALE = false>
static int launch(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int warps,
                  cudaStream_t stream, const GemvNorm& nrm = GemvNorm()) {
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(gemv_bf16_kernel<NT, TO, EPI, STAGES, SCALE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)gemv_smem(NT, STAGES, GEMV_MAX_WARPS));
    configured = true;
  }
  launch_pdl(gemv_bf16_kernel<NT, TO, EPI, STAGES, SCALE>, dim3(ceil_div(N, 16)), dim3(warps * 32),
             gemv_smem(NT, STAGES, warps), stream,
             static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
             static_cast<const __nv_bfloat16*>(bias), static_cast<TO*>(y), M, N, K, nrm);
  return launch_status("gemv_bf16");
}

// The warps of a block share its 16 rows' K blocks; fewer warps mean a smaller ring, so more blocks per SM: one
// block of 16 warps, three of 8, six of 4.  The largest block with which all blocks are on the GPU at once is
// taken (a second, partly filled wave costs its full length: the q/k/v projection's 432 blocks took 8.6 us as
// 296 + 136 and take 7.5 us as one wave); beyond 6 blocks per SM the smallest.  The choice depends on N and K
// only, never on M, so a row's result does not depend on its batch.
static int gemv_sm_count();
// Ring stages for NT row tiles.  Two tiles make four slots per stage: six stages would not fit 16 warps, and with
// 8 warps only two blocks an SM.
constexpr int gemv_stages(int nt) { return nt == 2 ? 4 : 6; }
static int gemv_shape(int M, int N, int K, int& warps, int& stages) {
  const int nt = M <= 8 ? 1 : 2;
  const int nblocks = (K + 31) / 32;
  const int ctas = ceil_div(N, 16);
  warps = ctas <= gemv_sm_count() ? 16 : (ctas <= 3 * gemv_sm_count() ? 8 : 4);
  while (warps > 1 && (warps / 2) * 2 >= nblocks) warps >>= 1;
  stages = gemv_stages(nt);
  return nt;
}

static int gemv_sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

}  // namespace exl3
