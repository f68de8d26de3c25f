// The entry point of the weight-streaming projection that takes part in a norm; the kernel is in gemv_bf16.cuh.
// A file of its own so that the two sets of kernel variants compile side by side.
#include "gemv_bf16.cuh"

using namespace exl3;

// The two sides of a norm that is no kernel of its own (see GemvNorm above).  Both take bfloat16 operands and
// at most 16 batch rows, as exl3_gemv_bf16.
//
// ss_in / ss_blocks / eps / width: when ss_in is not null, x is the x_raw of a producing call and the results are
// multiplied by rsqrt(sum of the blocks' sums / width + eps) per batch row before bias and gating.
// epilogue 0 or 1: y as in exl3_gemv_bf16 (out_dtype).  epilogue 2: no y; h[M, N] += result * rho,
// x_raw[M, N] = h * norm_w, ss_out[16, ceil(N / 16)] = the blocks' sums of squares.
extern "C" int exl3_gemv_bf16_normed(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M,
                                     int N, int K, int epilogue, const float* ss_in, int ss_blocks, float eps,
                                     float width, float* h, float rho, const void* norm_w, int norm_w_dtype,
                                     void* x_raw, float* ss_out, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 16 || N < 0 || K < 8 || K % 8 != 0 || epilogue < 0 || epilogue > 2 ||
      (epilogue == 1 && N % 16 != 0) || (ss_in != nullptr && (ss_blocks < 1 || !(width > 0.0f)))) {
    set_error("gemv_bf16_normed: bad arguments M=%d N=%d K=%d epilogue=%d ss_blocks=%d", M, N, K, epilogue, ss_blocks);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(x) || !aligned16(w)) { set_error("gemv_bf16_normed: x and w must be 16-byte aligned"); return ERR_ALIGNMENT; }
  GemvNorm nrm = {};
  if (epilogue == 2) {
    if (!h || !norm_w || !x_raw || !ss_out || (norm_w_dtype != DT_F32 && norm_w_dtype != DT_BF16)) {
      set_error("gemv_bf16_normed: the residual epilogue needs h, a float32 or bfloat16 norm weight, x_raw and ss_out");
      return ERR_BAD_ARGUMENT;
    }
    nrm.h = h;
    nrm.norm_w = norm_w;
    nrm.x_raw = static_cast<__nv_bfloat16*>(x_raw);
    nrm.ss_out = ss_out;
    nrm.rho = rho;
    nrm.norm_w_f32 = norm_w_dtype == DT_F32;
  } else if (out_dtype != DT_F32 && out_dtype != DT_BF16) {
    set_error("gemv_bf16_normed: unsupported output type %d", out_dtype);
    return ERR_UNSUPPORTED;
  }
  nrm.ss_in = ss_in;
  nrm.ss_blocks = ss_blocks;
  nrm.eps = eps;
  nrm.width = width;
  const bool f32 = out_dtype == DT_F32 && epilogue != 2;
  const bool scale = ss_in != nullptr;
  int warps, stages;
  const int nt = gemv_shape(M, N, K, warps, stages);
#define EXL3_GN4(NT, TO, EPI, ST)                                                                          \
  return scale ? launch<NT, TO, EPI, ST, true>(x, w, bias, y, M, N, K, warps, stream, nrm)                  \
               : launch<NT, TO, EPI, ST, false>(x, w, bias, y, M, N, K, warps, stream, nrm)
#define EXL3_GN3(NT, TO, EPI) { EXL3_GN4(NT, TO, EPI, gemv_stages(NT)); }   /* the ring's depth follows from NT */
#define EXL3_GN2(NT, EPI) if (f32) { EXL3_GN3(NT, float, EPI) } else { EXL3_GN3(NT, __nv_bfloat16, EPI) }
#define EXL3_GN1(NT) if (epilogue == 0) { EXL3_GN2(NT, 0) } else if (epilogue == 1) { EXL3_GN2(NT, 1) } else { EXL3_GN3(NT, __nv_bfloat16, 2) }
  if (nt == 1) { EXL3_GN1(1) }
  EXL3_GN1(2)
#undef EXL3_GN1
#undef EXL3_GN2
#undef EXL3_GN3
#undef EXL3_GN4
}
