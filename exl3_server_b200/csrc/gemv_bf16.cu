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
constexpr int GEMV_UNROLL = 6;      // 32-wide K blocks a warp has in flight

// EPI 0: y[m, n] = acc (+ bias).  EPI 1 (gated feed-forward): the 16 rows of a
// block are 8 gate rows followed by the 8 up rows of the same features;
// y[m, block * 8 + r] = silu(gate_r) * up_r, so N / 2 features come out.
template <int NT, typename TO, int EPI>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32)
gemv_bf16_kernel(const __nv_bfloat16* x, const __nv_bfloat16* __restrict__ w,
                 const __nv_bfloat16* __restrict__ bias, TO* __restrict__ y, int M, int N, int K) {
  __shared__ float part[GEMV_MAX_WARPS][16][8 * NT + 1];
  pdl_trigger();
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

  const int nblocks = (K + 31) / 32;
  bool waited = false;
  for (int kb0 = warp; kb0 < nblocks; kb0 += nwarps * GEMV_UNROLL) {
    // weights first: they do not depend on the kernel before this one
    uint4 a[GEMV_UNROLL], b[GEMV_UNROLL];
#pragma unroll
    for (int u = 0; u < GEMV_UNROLL; ++u) {
      const int k = (kb0 + u * nwarps) * 32 + tig * 8;
      const bool in = k < K;                          // K % 8 == 0: a piece is inside or outside
      a[u] = (in && ok_a) ? ldg_stream(wa + k) : zero;
      b[u] = (in && ok_b) ? ldg_stream(wb + k) : zero;
    }
    if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
    for (int u = 0; u < GEMV_UNROLL; ++u) {
      const int k = (kb0 + u * nwarps) * 32 + tig * 8;
      const bool in = k < K;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int m = t * 8 + gid;
        const uint4 xv = (in && m < M) ? __ldcg(reinterpret_cast<const uint4*>(x + (int64_t)m * K + k)) : zero;
        mma_bf16(c[t], a[u].x, b[u].x, a[u].y, b[u].y, xv.x, xv.y);
        mma_bf16(c[t], a[u].z, b[u].z, a[u].w, b[u].w, xv.z, xv.w);
      }
    }
  }
  if (!waited) pdl_wait();
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    part[warp][gid][t * 8 + tig * 2] = c[t][0];
    part[warp][gid][t * 8 + tig * 2 + 1] = c[t][1];
    part[warp][gid + 8][t * 8 + tig * 2] = c[t][2];
    part[warp][gid + 8][t * 8 + tig * 2 + 1] = c[t][3];
  }
  __syncthreads();
  if (EPI == 0) {
    for (int idx = threadIdx.x; idx < 16 * 8 * NT; idx += blockDim.x) {
      const int m = idx >> 4, r = idx & 15;           // consecutive threads: consecutive features
      const int n = r0 + r;
      if (m >= M || n >= N) continue;
      float s = 0.0f;
      for (int wi = 0; wi < nwarps; ++wi) s += part[wi][r][m];
      if (bias) s += __bfloat162float(bias[n]);
      Elem<TO>::store(y + (int64_t)m * N + n, s);
    }
  } else {
    const int n_out = N >> 1;
    for (int idx = threadIdx.x; idx < 8 * 8 * NT; idx += blockDim.x) {
      const int m = idx >> 3, r = idx & 7;
      const int f = blockIdx.x * 8 + r;
      if (m >= M || f >= n_out) continue;
      float g = 0.0f, u = 0.0f;
      for (int wi = 0; wi < nwarps; ++wi) { g += part[wi][r][m]; u += part[wi][r + 8][m]; }
      if (bias) { g += __bfloat162float(bias[r0 + r]); u += __bfloat162float(bias[r0 + r + 8]); }
      Elem<TO>::store(y + (int64_t)m * n_out + f, g / (1.0f + expf(-g)) * u);
    }
  }
}

template <int NT, typename TO, int EPI>
static int launch(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int warps,
                  cudaStream_t stream) {
  launch_pdl(gemv_bf16_kernel<NT, TO, EPI>, dim3(ceil_div(N, 16)), dim3(warps * 32), 0, stream,
             static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
             static_cast<const __nv_bfloat16*>(bias), static_cast<TO*>(y), M, N, K);
  return launch_status("gemv_bf16");
}

}  // namespace exl3

using namespace exl3;

// epilogue 0: plain; 1: silu(gate) * up over rows interleaved in eights (N even, N % 16 == 0)
extern "C" int exl3_gemv_bf16(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M,
                              int N, int K, int epilogue, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 16 || N < 0 || K < 8 || K % 8 != 0) {
    set_error("gemv_bf16: needs 1 <= M <= 16 and K a multiple of 8, got M=%d N=%d K=%d", M, N, K);
    return ERR_BAD_ARGUMENT;
  }
  if (epilogue != 0 && (epilogue != 1 || N % 16 != 0)) {
    set_error("gemv_bf16: the gated epilogue needs N a multiple of 16, got N=%d epilogue=%d", N, epilogue);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(x) || !aligned16(w)) { set_error("gemv_bf16: x and w must be 16-byte aligned"); return ERR_ALIGNMENT; }
  // Few blocks: many warps per block, so that one pass of GEMV_UNROLL K blocks
  // per warp covers K and every load is in flight at once.  Many blocks: fewer
  // warps each.  The choice depends on N and K only, never on M.
  const int nblocks = (K + 31) / 32;
  const int ctas = ceil_div(N, 16);
  int warps = ctas >= 8 * 148 ? 4 : (ctas >= 3 * 148 ? 8 : 16);
  while (warps > 1 && (warps / 2) * GEMV_UNROLL >= nblocks) warps >>= 1;
  const bool f32 = out_dtype == DT_F32;
  if (!f32 && out_dtype != DT_BF16) { set_error("gemv_bf16: unsupported output type %d", out_dtype); return ERR_UNSUPPORTED; }
#define EXL3_GEMV(NT, EPI)                                                                     \
  return f32 ? launch<NT, float, EPI>(x, w, bias, y, M, N, K, warps, stream)                   \
             : launch<NT, __nv_bfloat16, EPI>(x, w, bias, y, M, N, K, warps, stream)
  if (M <= 8) { if (epilogue) { EXL3_GEMV(1, 1); } else { EXL3_GEMV(1, 0); } }
  if (epilogue) { EXL3_GEMV(2, 1); } else { EXL3_GEMV(2, 0); }
#undef EXL3_GEMV
}
