// The plain entry point of the weight-streaming projection; the kernel is in gemv_bf16.cuh.
#include "gemv_bf16.cuh"

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
  const bool f32 = out_dtype == DT_F32;
  if (!f32 && out_dtype != DT_BF16) { set_error("gemv_bf16: unsupported output type %d", out_dtype); return ERR_UNSUPPORTED; }
  int warps, stages;
  const int nt = gemv_shape(M, N, K, warps, stages);
#define EXL3_GEMV(NT, EPI, ST)                                                                  \
  return f32 ? launch<NT, float, EPI, ST>(x, w, bias, y, M, N, K, warps, stream)                \
             : launch<NT, __nv_bfloat16, EPI, ST>(x, w, bias, y, M, N, K, warps, stream)
#define EXL3_GEMV_ST(NT, EPI) { EXL3_GEMV(NT, EPI, gemv_stages(NT)); }   /* the ring's depth follows from NT */
  if (nt == 1) { if (epilogue) { EXL3_GEMV_ST(1, 1) } else { EXL3_GEMV_ST(1, 0) } }
  if (epilogue) { EXL3_GEMV_ST(2, 1) } else { EXL3_GEMV_ST(2, 0) }
#undef EXL3_GEMV_ST
#undef EXL3_GEMV
}
