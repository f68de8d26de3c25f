// Decode-shaped projection: y[M,N] = x[M,K] . w[N,K]^T (+ bias) for M <= 16
// rows of x, bfloat16 operands, float32 accumulation.
//
// The weight matrix is read exactly once, in 16-byte pieces, straight from
// global memory into the A fragments of mma.m16n8k16 (weights are the 16-row
// operand, the batch is the 8-column one).  No shared-memory staging is
// needed because the order of the K index inside a 32-wide block is free: a
// thread's 8 consecutive weights and its 8 consecutive activations are
// assigned to the same logical k slots of two mma instructions.
//
// A block owns 16 output features; its warps take 32-wide K blocks in turn and
// their partial tiles are summed in warp order, so a result depends on K, N
// and the warp count only, never on M or the batch's other rows.
#include "api.h"
#include "common.cuh"

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

template <int NT, typename TO>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32)
gemv_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                 const __nv_bfloat16* __restrict__ bias, TO* __restrict__ y, int M, int N, int K) {
  __shared__ float part[GEMV_MAX_WARPS][16][8 * NT + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
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
  const uint4 zero = make_uint4(0, 0, 0, 0);

  constexpr int UNROLL = 4;
  const int nblocks = (K + 31) / 32;
  for (int kb0 = warp; kb0 < nblocks; kb0 += nwarps * UNROLL) {
    uint4 a[UNROLL], b[UNROLL], xv[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb0 + u * nwarps) * 32 + tig * 8;
      const bool in = k < K;                          // K % 8 == 0: a piece is inside or outside
      a[u] = (in && ok_a) ? ldg_stream(wa + k) : zero;
      b[u] = (in && ok_b) ? ldg_stream(wb + k) : zero;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int m = t * 8 + gid;
        xv[u][t] = (in && m < M) ? __ldg(reinterpret_cast<const uint4*>(x + (int64_t)m * K + k)) : zero;
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        mma_bf16(c[t], a[u].x, b[u].x, a[u].y, b[u].y, xv[u][t].x, xv[u][t].y);
        mma_bf16(c[t], a[u].z, b[u].z, a[u].w, b[u].w, xv[u][t].z, xv[u][t].w);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    part[warp][gid][t * 8 + tig * 2] = c[t][0];
    part[warp][gid][t * 8 + tig * 2 + 1] = c[t][1];
    part[warp][gid + 8][t * 8 + tig * 2] = c[t][2];
    part[warp][gid + 8][t * 8 + tig * 2 + 1] = c[t][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * 8 * NT; idx += blockDim.x) {
    const int m = idx >> 4, r = idx & 15;             // consecutive threads: consecutive features
    const int n = r0 + r;
    if (m >= M || n >= N) continue;
    float s = 0.0f;
    for (int wi = 0; wi < nwarps; ++wi) s += part[wi][r][m];
    if (bias) s += __bfloat162float(bias[n]);
    Elem<TO>::store(y + (int64_t)m * N + n, s);
  }
}

template <int NT, typename TO>
static int launch(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int warps,
                  cudaStream_t stream) {
  gemv_bf16_kernel<NT, TO><<<ceil_div(N, 16), warps * 32, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(bias), static_cast<TO*>(y), M, N, K);
  return launch_status("gemv_bf16");
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_gemv_bf16(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M,
                              int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 16 || N < 0 || K < 8 || K % 8 != 0) {
    set_error("gemv_bf16: needs 1 <= M <= 16 and K a multiple of 8, got M=%d N=%d K=%d", M, N, K);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(x) || !aligned16(w)) { set_error("gemv_bf16: x and w must be 16-byte aligned"); return ERR_ALIGNMENT; }
  // enough warps per block to keep loads in flight when there are few blocks; a
  // warp should still have at least one unrolled trip of K blocks
  const int nblocks = (K + 31) / 32;
  int warps = ceil_div(N, 16) >= 4 * 148 ? 4 : (ceil_div(N, 16) >= 2 * 148 ? 8 : 16);
  while (warps > 1 && warps * 4 > nblocks) warps >>= 1;
  const bool f32 = out_dtype == DT_F32;
  if (!f32 && out_dtype != DT_BF16) { set_error("gemv_bf16: unsupported output type %d", out_dtype); return ERR_UNSUPPORTED; }
  if (M <= 8) return f32 ? launch<1, float>(x, w, bias, y, M, N, K, warps, stream)
                         : launch<1, __nv_bfloat16>(x, w, bias, y, M, N, K, warps, stream);
  return f32 ? launch<2, float>(x, w, bias, y, M, N, K, warps, stream)
             : launch<2, __nv_bfloat16>(x, w, bias, y, M, N, K, warps, stream);
}
