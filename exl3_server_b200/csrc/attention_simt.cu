// Attention of query tokens over the paged key/value cache on the CUDA cores.
//
//   s[j] = (q . K[j]) * scale,  j in [max(0, pos - window + 1), pos]
//   out  = sum_j softmax(s)[j] * V[j]
//
// as in the reference's call of scaled-dot-product attention with an additive
// causal mask (src/model.cpp:539-548, 576-578); query head h reads key/value
// head h / (heads / kv_heads).  Scores, running maximum, running sum and the
// output accumulator are float32.
//
// One kernel serves whole prompts and single decoded tokens, in float32 and in
// bfloat16.  Work item: (token, kv head, chunk of split_keys keys).  A chunk is
// aligned to absolute positions, so the way keys are grouped, and therefore
// every rounding, depends only on the token's own position: not on the batch,
// not on how the tokens were cut into steps.  Inside a chunk the four warps
// take pages in turn; inside a warp each group of lanes owns the keys
// congruent to its index and keeps a private (max, sum, acc); the groups, the
// warps and the chunks are merged in a fixed order.  The chunks of a (token, kv
// head) are merged by whichever of their blocks finishes last (a counter at the
// start of the scratch memory tells it); the scratch must be zero when it is
// first used and is left with zero counters by every launch.
//
// Cache layout: pool[page][kv_head][slot][head_dim], page = block_table[row][pos / page_size].
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace exl3 {

constexpr int ATT_WARPS = 4;
constexpr int ATT_COUNTER_SLOTS = 65536;            // ints at the start of scratch, one per (token, kv head)

// The exponential of the softmax.  float32 path: expf on natural-log scores.
// bfloat16 path: scores are multiplied by log2(e) beforehand and ex2.approx is
// one instruction; maxima are then in base-2 units everywhere (registers,
// shared memory, scratch), consistently.
template <typename T> struct SoftmaxExp;
template <> struct SoftmaxExp<float> {
  static constexpr float prescale = 1.0f;
  __device__ static inline float exp(float x) { return expf(x); }
};
template <> struct SoftmaxExp<__nv_bfloat16> {
  static constexpr float prescale = 1.4426950408889634f;
  __device__ static inline float exp(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  }
};

// merge (mo, lo, ao) into (m, l, a)
template <typename T, int N>
__device__ inline void merge_state(float& m, float& l, float (&a)[N], float mo, float lo, const float (&ao)[N]) {
  const float mn = fmaxf(m, mo);
  if (mn == -INFINITY) return;                       // both empty
  const float cs = SoftmaxExp<T>::exp(m - mn), co = SoftmaxExp<T>::exp(mo - mn);
  l = l * cs + lo * co;
#pragma unroll
  for (int i = 0; i < N; ++i) a[i] = a[i] * cs + ao[i] * co;
  m = mn;
}

// Record layout in shared memory and scratch: [hd] accumulator, then max, then sum.
template <typename T, int GT, int R>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_tokens_kernel(const T* __restrict__ q, int64_t q_row_stride, T* __restrict__ out,
                   const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                   const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tok_pos,
                   const int* __restrict__ tok_seq, int nh, int nkv, int hd, int page, int window,
                   float scale, int split_keys, int max_splits, float* __restrict__ scratch,
                   int* __restrict__ counters, int lpk) {
  constexpr int VEC = Elem<T>::vec;
  constexpr int NA = R * VEC;
  constexpr int U = R == 1 ? 4 : 2;                  // key groups whose loads are issued together
  extern __shared__ float smem[];                    // [ATT_WARPS][GT][hd + 2], then [2][max_splits]
  __shared__ int is_last;
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, g = blockIdx.y, sp = blockIdx.z;
  const int G = nh / nkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kpw = 32 / lpk;                          // keys a warp handles at once
  const int grp = lane / lpk, li = lane - grp * lpk;
  const float scale_eff = scale * SoftmaxExp<T>::prescale;
  const int pos = __ldcg(tok_pos + t);
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int hi = pos + 1;
  // this block's chunk of keys
  int c_lo = lo, c_hi = hi;
  if (split_keys > 0) {
    const int c = lo / split_keys + sp;
    c_lo = max(lo, c * split_keys);
    c_hi = min(hi, (c + 1) * split_keys);
  }
  const int* bt = block_table + (int64_t)tok_seq[t] * bt_stride;
  const int rec = hd + 2;

  for (int h0 = 0; h0 < G; h0 += GT) {
    // this lane's slice of the queries
    float qv[GT][NA];
#pragma unroll
    for (int hh = 0; hh < GT; ++hh) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int d = (r * lpk + li) * VEC;
        float tmp[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) tmp[e] = 0.0f;
        if (d < hd && h0 + hh < G)
          load_vec_cg(q + (int64_t)t * q_row_stride + (int64_t)(g * G + h0 + hh) * hd + d, tmp);
#pragma unroll
        for (int e = 0; e < VEC; ++e) qv[hh][r * VEC + e] = tmp[e];
      }
    }
    float m[GT], l[GT], acc[GT][NA];
#pragma unroll
    for (int hh = 0; hh < GT; ++hh) {
      m[hh] = -INFINITY;
      l[hh] = 0.0f;
#pragma unroll
      for (int i = 0; i < NA; ++i) acc[hh][i] = 0.0f;
    }

    if (c_lo < c_hi) {
      const int first_page = c_lo / page, last_page = (c_hi - 1) / page;
      for (int pi = first_page + warp; pi <= last_page; pi += ATT_WARPS) {
        const int pg = bt[pi];
        const int64_t page_base = ((int64_t)pg * nkv + g) * page * hd;
        // U groups of keys at a time: all their loads are issued before the first is used
        for (int jj0 = grp; jj0 < page; jj0 += kpw * U) {   // same trip count for every lane
          uint4 rk[U][R], rv[U][R];
          bool valid[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int jj = jj0 + u * kpw;
            const int j = pi * page + jj;
            valid[u] = (jj < page) && (j >= c_lo) && (j < c_hi) && (pg >= 0);
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const int d = (r * lpk + li) * VEC;
              if (valid[u] && d < hd) {
                rk[u][r] = load_raw_cg(k_pool + page_base + (int64_t)jj * hd + d);
                rv[u][r] = load_raw_cg(v_pool + page_base + (int64_t)jj * hd + d);
              } else {
                rk[u][r] = make_uint4(0, 0, 0, 0);
                rv[u][r] = make_uint4(0, 0, 0, 0);
              }
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            float kv[NA], vv[NA];
#pragma unroll
            for (int r = 0; r < R; ++r) {
              float tk[VEC], tv[VEC];
              unpack_raw(rk[u][r], tk, (const T*)nullptr);
              unpack_raw(rv[u][r], tv, (const T*)nullptr);
#pragma unroll
              for (int e = 0; e < VEC; ++e) { kv[r * VEC + e] = tk[e]; vv[r * VEC + e] = tv[e]; }
            }
#pragma unroll
            for (int hh = 0; hh < GT; ++hh) {
              float s = 0.0f;
#pragma unroll
              for (int i = 0; i < NA; ++i) s = fmaf(qv[hh][i], kv[i], s);
              for (int o = lpk >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
              if (valid[u]) {
                s *= scale_eff;
                const float mn = fmaxf(m[hh], s);
                const float corr = SoftmaxExp<T>::exp(m[hh] - mn);    // exp(-inf) = 0 on the first key
                const float p = SoftmaxExp<T>::exp(s - mn);
                l[hh] = l[hh] * corr + p;
#pragma unroll
                for (int i = 0; i < NA; ++i) acc[hh][i] = acc[hh][i] * corr + p * vv[i];
                m[hh] = mn;
              }
            }
          }
        }
      }
    }
    // merge the lane groups of this warp (butterfly: both partners compute the same sum)
#pragma unroll
    for (int hh = 0; hh < GT; ++hh) {
      for (int o = lpk; o < 32; o <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m[hh], o);
        const float lo2 = __shfl_xor_sync(0xffffffffu, l[hh], o);
        float ao[NA];
#pragma unroll
        for (int i = 0; i < NA; ++i) ao[i] = __shfl_xor_sync(0xffffffffu, acc[hh][i], o);
        // keep the operand order the same on both partners
        if ((lane & o) == 0) {
          merge_state<T, NA>(m[hh], l[hh], acc[hh], mo, lo2, ao);
        } else {
          float m2 = mo, l2 = lo2;
          merge_state<T, NA>(m2, l2, ao, m[hh], l[hh], acc[hh]);
          m[hh] = m2; l[hh] = l2;
#pragma unroll
          for (int i = 0; i < NA; ++i) acc[hh][i] = ao[i];
        }
      }
    }
    __syncthreads();                                   // previous pass has read smem
    if (grp == 0) {
#pragma unroll
      for (int hh = 0; hh < GT; ++hh) {
        float* recp = smem + (warp * GT + hh) * rec;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int d = (r * lpk + li) * VEC;
          if (d < hd) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) recp[d + e] = acc[hh][r * VEC + e];
          }
        }
        if (li == 0) { recp[hd] = m[hh]; recp[hd + 1] = l[hh]; }
      }
    }
    __syncthreads();
    // merge the warps in order 0, 1, 2, 3; thread per (head, feature)
    for (int idx = threadIdx.x; idx < GT * hd; idx += blockDim.x) {
      const int hh = idx / hd, d = idx - hh * hd;
      if (h0 + hh >= G) continue;
      float mm = -INFINITY, ll = 0.0f, aa = 0.0f;
      for (int w = 0; w < ATT_WARPS; ++w) {
        const float* recp = smem + (w * GT + hh) * rec;
        const float mo = recp[hd], lo2 = recp[hd + 1];
        const float mn = fmaxf(mm, mo);
        if (mn == -INFINITY) continue;
        const float cs = SoftmaxExp<T>::exp(mm - mn), co = SoftmaxExp<T>::exp(mo - mn);
        ll = ll * cs + lo2 * co;
        aa = aa * cs + recp[d] * co;
        mm = mn;
      }
      const int head = g * G + h0 + hh;
      if (max_splits <= 1) {
        Elem<T>::store(out + ((int64_t)t * nh + head) * hd + d, aa / ll);
      } else {
        float* sc = scratch + (((int64_t)t * nh + head) * max_splits + sp) * rec;
        sc[d] = aa;
        if (d == 0) { sc[hd] = mm; sc[hd + 1] = ll; }
      }
    }
  }
  if (max_splits <= 1 || counters == nullptr) return;
  // The block that finishes last among the chunks of this (token, kv head) merges
  // them.  Which block that is varies; what it computes does not: the same sums
  // in chunk order.  The counter goes back to zero for the next launch.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(counters + (int64_t)t * nkv + g, 1) == max_splits - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float* sw = smem + ATT_WARPS * GT * rec;
  float* sl = sw + max_splits;
  for (int hq = 0; hq < G; ++hq) {
    const int head = g * G + hq;
    const float* base = scratch + ((int64_t)t * nh + head) * max_splits * rec;
    __syncthreads();
    for (int s2 = threadIdx.x; s2 < max_splits; s2 += blockDim.x) {
      sw[s2] = __ldcg(base + (int64_t)s2 * rec + hd);
      sl[s2] = __ldcg(base + (int64_t)s2 * rec + hd + 1);
    }
    __syncthreads();
    float mx = -INFINITY;
    for (int s2 = 0; s2 < max_splits; ++s2) mx = fmaxf(mx, sw[s2]);
    __syncthreads();
    for (int s2 = threadIdx.x; s2 < max_splits; s2 += blockDim.x) sw[s2] = SoftmaxExp<T>::exp(sw[s2] - mx);
    __syncthreads();
    float ll = 0.0f;
    for (int s2 = 0; s2 < max_splits; ++s2) ll += sl[s2] * sw[s2];
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
      float aa = 0.0f;
#pragma unroll 4
      for (int s2 = 0; s2 < max_splits; ++s2) aa += __ldcg(base + (int64_t)s2 * rec + d) * sw[s2];
      Elem<T>::store(out + ((int64_t)t * nh + head) * hd + d, aa / ll);
    }
  }
  if (threadIdx.x == 0) counters[(int64_t)t * nkv + g] = 0;
}

// out[t, head, :] from the per-chunk records.  With M the largest of the
// chunks' maxima and w_s = exp(m_s - M): out = sum_s acc_s w_s / sum_s l_s w_s,
// both sums in chunk order.  The records are read with independent loads.
template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ scratch, T* __restrict__ out, int nh, int hd,
                                    int max_splits) {
  extern __shared__ float sw[];                      // [max_splits] weights, then [max_splits] sums
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, head = blockIdx.y;
  const int rec = hd + 2;
  const float* base = scratch + ((int64_t)t * nh + head) * max_splits * rec;
  float* sl = sw + max_splits;
  for (int s = threadIdx.x; s < max_splits; s += blockDim.x) {
    sw[s] = __ldcg(base + (int64_t)s * rec + hd);
    sl[s] = __ldcg(base + (int64_t)s * rec + hd + 1);
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int s = 0; s < max_splits; ++s) mx = fmaxf(mx, sw[s]);
  __syncthreads();
  for (int s = threadIdx.x; s < max_splits; s += blockDim.x) sw[s] = SoftmaxExp<T>::exp(sw[s] - mx);   // empty chunk: exp(-inf) = 0
  __syncthreads();
  float ll = 0.0f;
  for (int s = 0; s < max_splits; ++s) ll += sl[s] * sw[s];
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float aa = 0.0f;
#pragma unroll 4
    for (int s = 0; s < max_splits; ++s) aa += __ldcg(base + (int64_t)s * rec + d) * sw[s];
    Elem<T>::store(out + ((int64_t)t * nh + head) * hd + d, aa / ll);
  }
}

template <typename T, int GT, int R>
static int launch_tokens(const void* q, int64_t q_row_stride, void* out, const void* k_pool,
                         const void* v_pool, const int* block_table, int bt_stride, const int* tok_pos,
                         const int* tok_seq, int T_, int nh, int nkv, int hd, int page, int window,
                         float scale, int split_keys, int max_splits, float* scratch, int lpk,
                         cudaStream_t stream) {
  const size_t smem = ((size_t)ATT_WARPS * GT * (hd + 2) + 2 * (size_t)max_splits) * sizeof(float);
  // The first ATT_COUNTER_BYTES of scratch are counters (zero between launches); records follow.
  // worth it only for a few tokens: with many, the merge kernel overlaps better than one block's loop
  const bool fused_merge = max_splits > 1 && T_ <= 2 && (int64_t)T_ * nkv <= ATT_COUNTER_SLOTS;
  int* counters = fused_merge ? reinterpret_cast<int*>(scratch) : nullptr;
  if (max_splits > 1) scratch = scratch + ATT_COUNTER_SLOTS;
  dim3 grid(T_, nkv, max_splits);
  launch_pdl(attn_tokens_kernel<T, GT, R>, grid, dim3(ATT_WARPS * 32), smem, stream,
             static_cast<const T*>(q), q_row_stride, static_cast<T*>(out), static_cast<const T*>(k_pool),
             static_cast<const T*>(v_pool), block_table, bt_stride, tok_pos, tok_seq, nh, nkv, hd, page, window,
             scale, split_keys, max_splits, scratch, counters, lpk);
  int rc = launch_status("attn_tokens");
  if (rc) return rc;
  if (max_splits > 1 && !fused_merge) {
    launch_pdl(attn_combine_kernel<T>, dim3(T_, nh), dim3(64), (size_t)2 * max_splits * sizeof(float), stream,
               (const float*)scratch, static_cast<T*>(out), nh, hd, max_splits);
    rc = launch_status("attn_combine");
  }
  return rc;
}

template <typename T>
static int dispatch(const void* q, int64_t q_row_stride, void* out, const void* k_pool, const void* v_pool,
                    const int* block_table, int bt_stride, const int* tok_pos, const int* tok_seq, int T_,
                    int nh, int nkv, int hd, int page, int window, float scale, int split_keys,
                    int max_splits, float* scratch, cudaStream_t stream) {
  constexpr int VEC = Elem<T>::vec;
  const int vecs = hd / VEC;                          // 16-byte pieces per head row
  int lpk = 1;
  while (lpk < vecs && lpk < 32) lpk <<= 1;
  const int R = ceil_div(vecs, lpk);
  const int G = nh / nkv;
#define EXL3_ATT(GT, RR)                                                                                 \
  return launch_tokens<T, GT, RR>(q, q_row_stride, out, k_pool, v_pool, block_table, bt_stride, tok_pos, \
                                  tok_seq, T_, nh, nkv, hd, page, window, scale, split_keys, max_splits, \
                                  scratch, lpk, stream)
  if (R == 1) {
    if (G == 1) EXL3_ATT(1, 1);
    if (G == 2) EXL3_ATT(2, 1);
    EXL3_ATT(4, 1);
  }
  if (R == 2) {
    if (G == 1) EXL3_ATT(1, 2);
    if (G == 2) EXL3_ATT(2, 2);
    EXL3_ATT(4, 2);
  }
#undef EXL3_ATT
  set_error("attn_tokens: head_dim %d is too large for this kernel", hd);
  return ERR_UNSUPPORTED;
}

}  // namespace exl3

using namespace exl3;

extern "C" size_t exl3_attn_tokens_scratch_bytes(int T, int nh, int hd, int max_splits) {
  if (max_splits <= 1) return 0;
  return (size_t)ATT_COUNTER_SLOTS * sizeof(int) + (size_t)T * nh * max_splits * (hd + 2) * sizeof(float);
}

extern "C" int exl3_attn_tokens(const void* q, int64_t q_row_stride, void* out, int dtype,
                                const void* k_pool, const void* v_pool, const int* block_table,
                                int bt_stride, const int* tok_pos, const int* tok_seq, int T, int nh, int nkv,
                                int hd, int page, int window, float scale, int split_keys, int max_splits,
                                float* scratch, size_t scratch_bytes, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || nh < 1 || nkv < 1 || nh % nkv != 0 || hd < 16 || hd % 16 != 0 || page < 1 || window < 0 ||
      max_splits < 1 || split_keys < 0 || (max_splits > 1 && split_keys == 0)) {
    set_error("attn_tokens: bad sizes T=%d heads=%d kv_heads=%d head_dim=%d (a multiple of 16) page=%d "
              "window=%d split_keys=%d max_splits=%d", T, nh, nkv, hd, page, window, split_keys, max_splits);
    return ERR_BAD_ARGUMENT;
  }
  if (split_keys % page != 0) {
    set_error("attn_tokens: split_keys %d must be a multiple of the page size %d", split_keys, page);
    return ERR_BAD_ARGUMENT;
  }
  if (nkv > 65535 || max_splits > 65535) { set_error("attn_tokens: grid too large"); return ERR_UNSUPPORTED; }
  const int vec = dtype == DT_F32 ? 4 : 8;
  if (!aligned16(q) || !aligned16(k_pool) || !aligned16(v_pool) || q_row_stride % vec != 0) {
    set_error("attn_tokens: q, k and v must be 16-byte aligned with a row stride in 16-byte units");
    return ERR_ALIGNMENT;
  }
  if (exl3_attn_tokens_scratch_bytes(T, nh, hd, max_splits) > scratch_bytes) {
    set_error("attn_tokens: scratch of %zu bytes is too small, need %zu", scratch_bytes,
              exl3_attn_tokens_scratch_bytes(T, nh, hd, max_splits));
    return ERR_SCRATCH;
  }
  if (dtype == DT_F32)
    return dispatch<float>(q, q_row_stride, out, k_pool, v_pool, block_table, bt_stride, tok_pos, tok_seq, T,
                           nh, nkv, hd, page, window, scale, split_keys, max_splits, scratch, stream);
  if (dtype == DT_BF16)
    return dispatch<__nv_bfloat16>(q, q_row_stride, out, k_pool, v_pool, block_table, bt_stride, tok_pos,
                                   tok_seq, T, nh, nkv, hd, page, window, scale, split_keys, max_splits,
                                   scratch, stream);
  set_error("attn_tokens: unsupported element type %d", dtype);
  return ERR_UNSUPPORTED;
}
