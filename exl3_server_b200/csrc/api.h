// C entry points of the kernel library.  Every function launches on the given
// stream and returns 0, a cudaError_t (> 0) or a negative code from
// common.cuh; exl3_last_error() gives the message of the calling thread's
// last failure.  Element type codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

extern "C" {

const char* exl3_last_error();
int exl3_abi_version();
long long exl3_launch_count();

int exl3_embed(const int* ids, const void* table, int table_dtype, float* h, int T, int H, int V,
               float scale, cudaStream_t stream);
int exl3_add_rmsnorm(float* h, const void* y, int y_dtype, float y_scale, const void* w, int w_dtype,
                     float eps, void* out, int out_dtype, float out_scale, const int* rows, int n_rows,
                     int H, cudaStream_t stream);
// interleave 0: gu = [gate (I) | up (I)]; 8: eight gate columns, then the eight up columns of the same features.
int exl3_silu_mul(const void* gu, void* out, int dtype, int T, int I, int interleave, cudaStream_t stream);
// inv_freq: rot / 2 frequencies; inv_freq_lo: what float32 lost of them, or null (see rope_sincos in common.cuh).
int exl3_rope_kv_write(void* qkv, int dtype, const float* inv_freq, const float* inv_freq_lo, int rot,
                       float pos_scale, const int* tok_pos, const int* tok_seq, const int* block_table, int bt_stride,
                       void* k_pool, void* v_pool, int T, int nh, int nkv, int hd, int page, int write_kv,
                       cudaStream_t stream);

// y[M,N] = x[M,K] . w[N,K]^T (+ bias[N]); any sizes; float32 accumulation in a
// fixed order over K.  in_dtype covers x, w and bias; out_dtype covers y.
int exl3_gemm_simt(const void* x, const void* w, const void* bias, void* y, int in_dtype, int out_dtype,
                   int M, int N, int K, cudaStream_t stream);
// bfloat16 weights streamed once for M <= 16 rows of x (tensor-core mma, K % 8 == 0).
// epilogue 1: rows of w are 8 gate rows then 8 up rows, repeated; y[M, N/2] = silu(gate) * up.
int exl3_gemv_bf16(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N,
                   int K, int epilogue, cudaStream_t stream);

// bfloat16 GEMM on tcgen05 tensor cores with TMA loads (K and N multiples of 8); epilogue 1 as in
// exl3_gemv_bf16 (N a multiple of 16, output N/2 wide).  exl3_gemm_tc_status() returns and clears the
// code a kernel left when one of its bounded waits ran out (0: none).
int exl3_gemm_tc(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int epilogue,
                 cudaStream_t stream);
int exl3_gemm_tc_status();
// Launches a kernel whose only wait can never be satisfied (short limit): status becomes 9.
int exl3_gemm_tc_wait_selftest(cudaStream_t stream);

// Attention of single query tokens over the paged cache.  Token t belongs to
// batch row tok_seq[t] and sits at position tok_pos[t]; it sees keys
// max(0, pos - window + 1) .. pos (window 0: from 0).  n_splits > 1 cuts the
// keys into chunks of split_keys and needs scratch; see attention_simt.cu.
int exl3_attn_tokens(const void* q, int64_t q_row_stride, void* out, int dtype, const void* k_pool,
                     const void* v_pool, const int* block_table, int bt_stride, const int* tok_pos,
                     const int* tok_seq, int T, int nh, int nkv, int hd, int page, int window, float scale,
                     int split_keys, int max_splits, float* scratch, size_t scratch_bytes,
                     cudaStream_t stream);
size_t exl3_attn_tokens_scratch_bytes(int T, int nh, int hd, int max_splits);

size_t exl3_argmax_scratch_bytes(int R, int V);
// Whole prompts on tcgen05 tensor cores with TMA loads from the paged cache (bfloat16, heads of 64 or 128, pages
// of 64, tiles of 128 queries); variant 0: chosen by the number of blocks, 1: a tile a block, 2: four blocks an SM
// (heads of 64), 3: two tiles a block (the first of the list with the last, and so on); see attention_prefill_tc.cu.
int exl3_attn_prefill_tc_supported(int dtype, int hd, int page);
int exl3_attn_prefill_tc_status();
int exl3_attn_prefill_tc(const void* q, int64_t q_row_stride, int T, void* out, const void* k_pool,
                         const void* v_pool, int64_t n_pool_rows, const int* block_table, int bt_stride,
                         const int* row_start, const int* row_pos0, const int* tile_seq, const int* tile_q0,
                         int n_tiles, int nh, int nkv, int hd, int page, int window, float scale, int variant,
                         cudaStream_t stream);

// exl3_gemv_bf16 as the two sides of a norm that is no kernel of its own.  With ss_in the input is the x_raw of a
// producing call and the results are multiplied by rsqrt(sum of ss_in's blocks / width + eps) per batch row.
// With epilogue 2 no y is written: h[M, N] += result * rho, x_raw = h * norm_w, ss_out[16, ceil(N / 16)] = sums of
// squares per batch row and block.  See gemv_bf16.cuh.
int exl3_gemv_bf16_normed(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N,
                          int K, int epilogue, const float* ss_in, int ss_blocks, float eps, float width, float* h,
                          float rho, const void* norm_w, int norm_w_dtype, void* x_raw, float* ss_out,
                          cudaStream_t stream);

// The same projection and epilogues for up to 128 rows on tcgen05 tensor cores: the weights are the 128-row operand
// and stream once by TMA, K is cut over the blocks of a cluster and summed through distributed shared memory (no
// scratch, no atomics).  ss_in / ss_out are [rows >= M, blocks].  split: cuts of K, 0 = chosen from N and K; tiles:
// 128-row tiles of w per block (1 or 2), 0 = chosen.
// exl3_gemm_skinny_status() returns and clears the code a kernel left when one of its bounded waits ran out.
int exl3_gemm_skinny(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N, int K,
                     int epilogue, const float* ss_in, int ss_blocks, float eps, float width, float* h, float rho,
                     const void* norm_w, int norm_w_dtype, void* x_raw, float* ss_out, int split, int tiles,
                     cudaStream_t stream);
int exl3_gemm_skinny_status();
int exl3_gemm_skinny_max_rows();
int exl3_gemm_skinny_split(int N, int K);
int exl3_gemm_skinny_max_clusters(int s);

// Projections of many rows with two blocks of a cluster as one tensor core (tcgen05.mma.cta_group::2, tiles of
// 256 x 256): input and epilogues as exl3_gemm_skinny's (0 plain, 1 gated, 2 residual and the next norm's pieces),
// y bfloat16; ss_out is [M, exl3_gemm_pair_ss_blocks(N)].  exl3_gemm_pair_status() returns and clears the code a
// kernel left when one of its bounded waits ran out.
int exl3_gemm_pair(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int epilogue,
                   const float* ss_in, int ss_blocks, float eps, float width, float* h, float rho,
                   const void* norm_w, int norm_w_dtype, void* x_raw, float* ss_out, cudaStream_t stream);
// The q/k/v projection of heads of 64 with the half-split rotary encoding (rot 64, or 0 for none) and the cache
// write in its epilogue: of y [M, (nh + 2 nkv) * 64] only the queries' columns are written; rotated keys and
// values go to each token's place in the paged pools (write_kv).
int exl3_gemm_pair_rope(const void* x, const void* w, const void* bias, void* y, int M, int K, const float* ss_in,
                        int ss_blocks, float eps, float width, const int* tok_pos, const int* tok_seq,
                        const int* block_table, int bt_stride, const float* inv_freq, const float* inv_freq_lo, int rot,
                        float pos_scale, int nh, int nkv, int hd, int page, void* k_pool, void* v_pool,
                        int64_t pool_rows, int write_kv, cudaStream_t stream);
int exl3_gemm_pair_status();
int exl3_gemm_pair_ss_blocks(int N);

// Decoded tokens on the tensor cores with TMA loads from the paged cache (bfloat16, head_dim 64 or 128, pages of 64, up
// to 16 query heads per kv head, 1024 tokens, 256 chunks); arguments and scratch as exl3_attn_tokens; optionally
// it applies the rotary encoding and takes each token's own key and value from the projection's output, writing
// them to the cache itself.  head_split n (a divisor of the query heads per kv head): the query heads of a kv head
// as n groups of work.  in_block 1: a block per (token, group of heads), whose warps take the item's chunks (at most
// 4) and merge them in shared memory; 2: a cluster of two blocks (at most 8 chunks, the first block merging, the
// second one's records read out of its shared memory); no scratch in either.  twins 2 (with in_block 1 or 2, an even
// head_split and groups of up to 8 heads): two groups of query heads of a kv head per block, walking the same pages
// out of the same rings, 8 computing warps.  See attention_decode.cu.
int exl3_attn_decode_supported(int dtype, int T, int nh, int nkv, int hd, int page, int split_keys, int max_splits);
int exl3_attn_decode_status();
int exl3_attn_decode(const void* q, int64_t q_row_stride, void* out, void* k_pool, void* v_pool,
                     int64_t n_pool_rows, const int* block_table, int bt_stride, const int* tok_pos,
                     const int* tok_seq, int T, int nh, int nkv, int hd, int page, int window, float scale,
                     int split_keys, int max_splits, float* scratch, size_t scratch_bytes, const float* inv_freq,
                     const float* inv_freq_lo, int rot, float pos_scale, int write_new, int head_split, int in_block,
                     int twins, cudaStream_t stream);

int exl3_argmax(const float* logits, int* out, int R, int V, void* scratch, size_t scratch_bytes,
                cudaStream_t stream);
// The reference's sampler on the device (see sampling_filtered.cu).  rows: float64 [R, 5] = temperature (<= 0:
// greedy), top_k (0: off; at most exl3_sample_filtered_cap()), top_p, min_p, uniform number in [0, 1).
int exl3_sample_filtered(const float* logits, const double* rows, int* out, int R, int V, cudaStream_t stream);
int exl3_sample_filtered_cap();
// counts: R device pointers (null: none) to int32 [V] token counts of the rows' contexts; params: float32 [R, 3] =
// repetition, presence and frequency penalty.  Changes logits in place.  exl3_sample_count adds the chosen tokens.
int exl3_sample_penalties(float* logits, int R, int V, const int* const* counts, const float* params,
                          cudaStream_t stream);
int exl3_sample_count(int* const* counts, const int* ids, int R, int V, cudaStream_t stream);
}
