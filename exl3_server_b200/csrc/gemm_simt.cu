// Plain matrix product on the CUDA cores: y[M,N] = x[M,K] . w[N,K]^T (+ bias).
//
// This is the true 32-bit path of every projection (no tensor cores, no
// reduced-precision mode) and the fallback for sizes the fast kernels refuse.
// Each output element is one float32 accumulator that walks K from 0 upward,
// so its value does not depend on M, N, the tiling or what else is in the
// batch.  The reference keeps weights as (in, out) and calls a library matmul
// (src/model.cpp:549-552); the checkpoint's (out, in) order is kept here.
#include "api.h"
#include "common.cuh"

namespace exl3 {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TI* __restrict__ x, const TI* __restrict__ w, const TI* __restrict__ bias,
                 TO* __restrict__ y, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;            // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k per operand: thread loads 4 elements of each
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      float a = 0.0f, b = 0.0f;
      if (k < K) {
        if (m0 + r < M) a = Elem<TI>::load(x + (int64_t)(m0 + r) * K + k);
        if (n0 + r < N) b = Elem<TI>::load(w + (int64_t)(n0 + r) * K + k);
      }
      As[kk][r] = a;
      Bs[kk][r] = b;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += Elem<TI>::load(bias + n);
      Elem<TO>::store(y + (int64_t)m * N + n, v);
    }
  }
}

template <typename TI, typename TO>
static int launch(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                  cudaStream_t stream) {
  dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
  if (grid.y > 65535) { set_error("gemm_simt: M=%d is too large", M); return ERR_UNSUPPORTED; }
  gemm_simt_kernel<TI, TO><<<grid, 256, 0, stream>>>(static_cast<const TI*>(x), static_cast<const TI*>(w),
                                                      static_cast<const TI*>(bias), static_cast<TO*>(y), M, N, K);
  return launch_status("gemm_simt");
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_gemm_simt(const void* x, const void* w, const void* bias, void* y, int in_dtype,
                              int out_dtype, int M, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || N < 0 || K < 1) { set_error("gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K); return ERR_BAD_ARGUMENT; }
  if (in_dtype == DT_F32 && out_dtype == DT_F32) return launch<float, float>(x, w, bias, y, M, N, K, stream);
  if (in_dtype == DT_BF16 && out_dtype == DT_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16>(x, w, bias, y, M, N, K, stream);
  if (in_dtype == DT_BF16 && out_dtype == DT_F32) return launch<__nv_bfloat16, float>(x, w, bias, y, M, N, K, stream);
  set_error("gemm_simt: unsupported element types in=%d out=%d", in_dtype, out_dtype);
  return ERR_UNSUPPORTED;
}
