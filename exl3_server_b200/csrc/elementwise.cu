// Memory-bound parts of the step: embedding gather with scale, fused
// residual-add + RMSNorm, SiLU(gate)*up, rotary position encoding fused with
// the write of keys and values into the paged cache.
//
// Formulas follow the reference's forward pass (src/model.cpp:529 gather,
// :556/:582/:589 RMSNorm, :566-574 rotation then cache append, :585-586
// SiLU*up); statistics, angles and the residual sum are computed in float32.
#include "api.h"
#include "common.cuh"

namespace exl3 {

__device__ inline float load_any(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? static_cast<const float*>(p)[i]
                         : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
// for data that an earlier kernel of the same step wrote (see load_vec_cg)
__device__ inline float load_act(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
}
__device__ inline void store_any(void* p, int dtype, int64_t i, float v) {
  if (dtype == DT_F32) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// h[t,:] = table[ids[t],:] * scale
__global__ void embed_kernel(const int* __restrict__ ids, const void* __restrict__ table,
                             int table_dtype, float* __restrict__ h, int H, int V, float scale) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int id = __ldcg(ids + t);
  float* row = h + (int64_t)t * H;
  if (id < 0 || id >= V) {                       // refused on the host already; never read outside
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = 0.0f;
    return;
  }
  const int64_t base = (int64_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = load_any(table, table_dtype, base + i) * scale;
}

// For each listed row r (all rows when rows == nullptr):
//   h[r,:] += y[r,:] * y_scale            (skipped when y == nullptr)
//   out[i,:] = h[r,:] * rsqrt(mean(h[r,:]^2) + eps) * w * out_scale
// i is the index in the list, so the output is compact.
__global__ void add_rmsnorm_kernel(float* h, const void* y, int y_dtype,
                                   float y_scale, const void* __restrict__ w, int w_dtype, float eps,
                                   void* __restrict__ out, int out_dtype, float out_scale,
                                   const int* __restrict__ rows, int H) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* hr = h + (int64_t)r * H;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = __ldcg(hr + c);
    if (y) {
      v += load_act(y, y_dtype, (int64_t)r * H + c) * y_scale;
      hr[c] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = __ldcg(hr + c) * inv * load_any(w, w_dtype, c) * out_scale;   // same thread wrote hr[c]
    store_any(out, out_dtype, (int64_t)i * H + c, v);
  }
}

// The same for rows of up to NORM_THREADS * 4 * NORM_VECS values with H % 8 == 0
// and 16-bit y / out: a thread keeps its pieces of the row in registers, so h
// and y are read once, with all loads in flight together.
constexpr int NORM_THREADS = 256;
constexpr int NORM_VECS = 4;                     // pieces of 8 values per thread: rows up to 8192

template <typename WT>
__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_bf16_kernel(float* h, const __nv_bfloat16* y, float y_scale, const WT* __restrict__ w, float eps,
                        __nv_bfloat16* out, float out_scale, const int* __restrict__ rows, int H) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* hr = h + (int64_t)r * H;
  const __nv_bfloat16* yr = y ? y + (int64_t)r * H : nullptr;
  float v[NORM_VECS][8];
  float ss = 0.0f;
#pragma unroll
  for (int p = 0; p < NORM_VECS; ++p) {
    const int c = (p * NORM_THREADS + threadIdx.x) * 8;
    if (c < H) {
      float a[4], b[4];
      load_vec_cg(hr + c, a);
      load_vec_cg(hr + c + 4, b);
#pragma unroll
      for (int e = 0; e < 4; ++e) { v[p][e] = a[e]; v[p][4 + e] = b[e]; }
    }
  }
  if (yr) {
#pragma unroll
    for (int p = 0; p < NORM_VECS; ++p) {
      const int c = (p * NORM_THREADS + threadIdx.x) * 8;
      if (c < H) {
        float yy[8];
        load_vec_cg(yr + c, yy);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[p][e] += yy[e] * y_scale;
        const float a[4] = {v[p][0], v[p][1], v[p][2], v[p][3]}, b[4] = {v[p][4], v[p][5], v[p][6], v[p][7]};
        store_vec(hr + c, a);
        store_vec(hr + c + 4, b);
      }
    }
  }
#pragma unroll
  for (int p = 0; p < NORM_VECS; ++p) {
    const int c = (p * NORM_THREADS + threadIdx.x) * 8;
    if (c < H) {
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[p][e] * v[p][e];
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int p = 0; p < NORM_VECS; ++p) {
    const int c = (p * NORM_THREADS + threadIdx.x) * 8;
    if (c < H) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[p][e] * inv * Elem<WT>::load(w + c + e) * out_scale;
      store_vec(out + (int64_t)i * H + c, o);
    }
  }
}

// out[t,i] = silu(gate[t,i]) * up[t,i].  interleave 0: gu[t] = [gate (I) | up (I)];
// interleave 8: gu[t] = eight gate columns, the eight up columns of the same
// features, and so on (the layout the fused decode projection's weights have).
__global__ void silu_mul_kernel(const void* __restrict__ gu, void* __restrict__ out, int dtype,
                                int64_t total, int I, int interleave) {
  pdl_wait();
  pdl_trigger();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t t = idx / I;
  const int i = (int)(idx - t * I);
  int64_t gi, ui;
  if (interleave == 0) {
    gi = t * 2 * I + i;
    ui = gi + I;
  } else {
    gi = t * 2 * I + (int64_t)(i / interleave) * 2 * interleave + (i % interleave);
    ui = gi + interleave;
  }
  const float g = load_act(gu, dtype, gi);
  const float u = load_act(gu, dtype, ui);
  store_any(out, dtype, idx, g / (1.0f + expf(-g)) * u);
}

// The same with 16-byte accesses: a thread makes VEC outputs (I % VEC == 0, and
// an interleave that is a multiple of VEC).
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_vec_kernel(const T* gu, T* out, int64_t total_vecs, int I, int interleave) {
  constexpr int VEC = Elem<T>::vec;
  pdl_wait();
  pdl_trigger();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_vecs) return;
  const int per_row = I / VEC;
  const int64_t t = idx / per_row;
  const int i0 = (int)(idx - t * per_row) * VEC;
  const int64_t go = t * 2 * I + (interleave == 0 ? i0 : (i0 / interleave) * 2 * interleave + (i0 % interleave));
  const int64_t uo = go + (interleave == 0 ? I : interleave);
  float g[VEC], u[VEC], o[VEC];
  load_vec_cg(gu + go, g);
  load_vec_cg(gu + uo, u);
#pragma unroll
  for (int e = 0; e < VEC; ++e) o[e] = g[e] / (1.0f + expf(-g[e])) * u[e];
  store_vec(out + t * I + i0, o);
}

// One block per token.  qkv[t] = [q heads | k heads | v heads], each head_dim
// wide.  q and k are rotated in place (half-split pairs d, d + rot/2 with
// angle pos * pos_scale * (inv_freq[d] + inv_freq_lo[d])); rotated k and plain v are written to
// the token's place in the paged cache.
__global__ void rope_kv_write_kernel(void* __restrict__ qkv, int dtype, const float* __restrict__ inv_freq,
                                     const float* __restrict__ inv_freq_lo, int rot, float pos_scale, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                     int bt_stride, void* __restrict__ k_pool, void* __restrict__ v_pool,
                                     int nh, int nkv, int hd, int page, int write_kv) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = rot >> 1;
  const int row = (nh + 2 * nkv) * hd;
  const int64_t base = (int64_t)t * row;
  int64_t cache_base = 0;
  bool cache_ok = false;
  if (write_kv) {
    const int pg = block_table[(int64_t)tok_seq[t] * bt_stride + pos / page];
    cache_ok = pg >= 0;
    cache_base = ((int64_t)pg * nkv * page + (pos % page)) * hd;   // + g * page * hd
  }
  const float p = (float)pos * pos_scale;
  // rotated pairs of q and k: a thread keeps one pair index d, computes its sine
  // and cosine once and walks over the heads
  const int n_rot_heads = nh + nkv;
  auto rotate_heads = [&](int d, int first, int step) {
    float s, c;
    rope_sincos(p, inv_freq[d], inv_freq_lo ? inv_freq_lo[d] : 0.0f, &s, &c);
    for (int head = first; head < n_rot_heads; head += step) {
      const int64_t a = base + (int64_t)head * hd + d;
      const float x0 = load_act(qkv, dtype, a), x1 = load_act(qkv, dtype, a + half);
      const float r0 = x0 * c - x1 * s, r1 = x1 * c + x0 * s;
      if (head < nh) {
        store_any(qkv, dtype, a, r0);
        store_any(qkv, dtype, a + half, r1);
      } else if (cache_ok) {
        const int64_t ca = cache_base + (int64_t)(head - nh) * page * hd + d;
        store_any(k_pool, dtype, ca, r0);
        store_any(k_pool, dtype, ca + half, r1);
      }
    }
  };
  if (half > 0 && (int)blockDim.x >= half) {
    const int lanes = blockDim.x / half;              // groups of threads that share the heads
    if ((int)threadIdx.x < lanes * half) rotate_heads(threadIdx.x % half, threadIdx.x / half, lanes);
  } else if (half > 0) {
    for (int d = threadIdx.x; d < half; d += blockDim.x) rotate_heads(d, 0, 1);
  }
  if (!cache_ok) return;
  // features of k beyond the rotated ones pass through
  const int tail = hd - rot;
  for (int i = threadIdx.x; i < nkv * tail; i += blockDim.x) {
    const int g = i / tail, d = rot + (i - g * tail);
    store_any(k_pool, dtype, cache_base + (int64_t)g * page * hd + d,
              load_act(qkv, dtype, base + (int64_t)(nh + g) * hd + d));
  }
  for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x) {
    const int g = i / hd, d = i - g * hd;
    store_any(v_pool, dtype, cache_base + (int64_t)g * page * hd + d,
              load_act(qkv, dtype, base + (int64_t)(nh + nkv + g) * hd + d));
  }
}

// The same with 16-byte accesses: a work item is one head's piece of VEC
// features in the first half together with its partner piece in the second
// half (then the pass-through pieces of k, then the pieces of v).  Needs
// rot % (2 VEC) == 0 and hd % VEC == 0.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_write_vec_kernel(T* qkv, const float* __restrict__ inv_freq, const float* __restrict__ inv_freq_lo, int rot,
                         float pos_scale,
                         const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                         const int* __restrict__ block_table, int bt_stride, T* k_pool, T* v_pool, int nh, int nkv,
                         int hd, int page, int write_kv) {
  constexpr int VEC = Elem<T>::vec;
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int pos = __ldcg(tok_pos + t);
  const int half = rot >> 1;
  const int64_t base = (int64_t)t * (nh + 2 * nkv) * hd;
  int64_t cache_base = 0;
  bool cache_ok = false;
  if (write_kv) {
    const int pg = block_table[(int64_t)__ldcg(tok_seq + t) * bt_stride + pos / page];
    cache_ok = pg >= 0;
    cache_base = ((int64_t)pg * nkv * page + (pos % page)) * hd;
  }
  const float p = (float)pos * pos_scale;
  // the token's sines and cosines, once for all its heads
  extern __shared__ float rope_cs[];                  // [half] cosines, then [half] sines
  for (int d = threadIdx.x; d < half; d += blockDim.x)
    rope_sincos(p, inv_freq[d], inv_freq_lo ? inv_freq_lo[d] : 0.0f, &rope_cs[half + d], &rope_cs[d]);
  __syncthreads();
  const int cpr = half / VEC;                         // rotated pieces per head (first half)
  const int n_rot = (nh + nkv) * cpr;
  const int tail = (hd - rot) / VEC;                  // pass-through pieces per k head
  const int n_tail = cache_ok ? nkv * tail : 0;
  const int n_v = cache_ok ? nkv * (hd / VEC) : 0;
  for (int i = threadIdx.x; i < n_rot + n_tail + n_v; i += blockDim.x) {
    if (i < n_rot) {
      const int head = i / cpr, d = (i - head * cpr) * VEC;
      float x0[VEC], x1[VEC], r0[VEC], r1[VEC];
      T* src = qkv + base + (int64_t)head * hd + d;
      load_vec_cg(src, x0);
      load_vec_cg(src + half, x1);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float c = rope_cs[d + e], s = rope_cs[half + d + e];
        r0[e] = x0[e] * c - x1[e] * s;
        r1[e] = x1[e] * c + x0[e] * s;
      }
      if (head < nh) {
        store_vec(src, r0);
        store_vec(src + half, r1);
      } else if (cache_ok) {
        T* dst = k_pool + cache_base + (int64_t)(head - nh) * page * hd + d;
        store_vec(dst, r0);
        store_vec(dst + half, r1);
      }
    } else if (i < n_rot + n_tail) {
      const int j = i - n_rot;
      const int g = j / tail, d = rot + (j - g * tail) * VEC;
      float x[VEC];
      load_vec_cg(qkv + base + (int64_t)(nh + g) * hd + d, x);
      store_vec(k_pool + cache_base + (int64_t)g * page * hd + d, x);
    } else {
      const int j = i - n_rot - n_tail;
      const int g = j / (hd / VEC), d = (j - g * (hd / VEC)) * VEC;
      float x[VEC];
      load_vec_cg(qkv + base + (int64_t)(nh + nkv + g) * hd + d, x);
      store_vec(v_pool + cache_base + (int64_t)g * page * hd + d, x);
    }
  }
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_embed(const int* ids, const void* table, int table_dtype, float* h, int T, int H,
                          int V, float scale, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H < 1 || V < 1) { set_error("embed: bad sizes T=%d H=%d V=%d", T, H, V); return ERR_BAD_ARGUMENT; }
  launch_pdl(embed_kernel, dim3(T), dim3(256), 0, stream, ids, table, table_dtype, h, H, V, scale);
  return launch_status("embed");
}

extern "C" int exl3_add_rmsnorm(float* h, const void* y, int y_dtype, float y_scale, const void* w,
                                int w_dtype, float eps, void* out, int out_dtype, float out_scale,
                                const int* rows, int n_rows, int H, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  if (n_rows < 0 || H < 1) { set_error("add_rmsnorm: bad sizes rows=%d H=%d", n_rows, H); return ERR_BAD_ARGUMENT; }
  const bool fast = out_dtype == DT_BF16 && (y == nullptr || y_dtype == DT_BF16) && H % 8 == 0 &&
                    H <= NORM_THREADS * 8 * NORM_VECS && aligned16(h) && aligned16(out) && aligned16(y);
  if (fast && w_dtype == DT_BF16) {
    launch_pdl(add_rmsnorm_bf16_kernel<__nv_bfloat16>, dim3(n_rows), dim3(NORM_THREADS), 0, stream, h,
               static_cast<const __nv_bfloat16*>(y), y_scale, static_cast<const __nv_bfloat16*>(w), eps,
               static_cast<__nv_bfloat16*>(out), out_scale, rows, H);
  } else if (fast) {
    launch_pdl(add_rmsnorm_bf16_kernel<float>, dim3(n_rows), dim3(NORM_THREADS), 0, stream, h,
               static_cast<const __nv_bfloat16*>(y), y_scale, static_cast<const float*>(w), eps,
               static_cast<__nv_bfloat16*>(out), out_scale, rows, H);
  } else {
    launch_pdl(add_rmsnorm_kernel, dim3(n_rows), dim3(256), 0, stream, h, y, y_dtype, y_scale, w, w_dtype, eps, out,
               out_dtype, out_scale, rows, H);
  }
  return launch_status("add_rmsnorm");
}

extern "C" int exl3_silu_mul(const void* gu, void* out, int dtype, int T, int I, int interleave,
                             cudaStream_t stream) {
  const int64_t total = (int64_t)T * I;
  if (total == 0) return 0;
  if (T < 0 || I < 1 || interleave < 0 || (interleave > 0 && I % interleave != 0)) {
    set_error("silu_mul: bad sizes T=%d I=%d interleave=%d", T, I, interleave);
    return ERR_BAD_ARGUMENT;
  }
  const int64_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) { set_error("silu_mul: too many elements"); return ERR_UNSUPPORTED; }
  const int vec = dtype == DT_F32 ? 4 : 8;
  if (I % vec == 0 && interleave % vec == 0 && aligned16(gu) && aligned16(out)) {
    const int64_t vecs = total / vec;
    const unsigned vblocks = (unsigned)((vecs + 255) / 256);
    if (dtype == DT_F32)
      launch_pdl(silu_mul_vec_kernel<float>, dim3(vblocks), dim3(256), 0, stream, static_cast<const float*>(gu),
                 static_cast<float*>(out), vecs, I, interleave);
    else
      launch_pdl(silu_mul_vec_kernel<__nv_bfloat16>, dim3(vblocks), dim3(256), 0, stream,
                 static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), vecs, I, interleave);
    return launch_status("silu_mul");
  }
  launch_pdl(silu_mul_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, gu, out, dtype, total, I, interleave);
  return launch_status("silu_mul");
}

extern "C" int exl3_rope_kv_write(void* qkv, int dtype, const float* inv_freq, const float* inv_freq_lo, int rot,
                                  float pos_scale,
                                  const int* tok_pos, const int* tok_seq, const int* block_table,
                                  int bt_stride, void* k_pool, void* v_pool, int T, int nh, int nkv, int hd,
                                  int page, int write_kv, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || nh < 1 || nkv < 1 || hd < 2 || page < 1 || rot < 0 || rot > hd || (rot & 1)) {
    set_error("rope_kv_write: bad sizes T=%d heads=%d kv_heads=%d head_dim=%d rot=%d page=%d", T, nh, nkv,
              hd, rot, page);
    return ERR_BAD_ARGUMENT;
  }
  const int vec = dtype == DT_F32 ? 4 : 8;
  const bool fast = rot % (2 * vec) == 0 && hd % vec == 0 && aligned16(qkv) && aligned16(k_pool) && aligned16(v_pool);
  if (fast && dtype == DT_F32) {
    launch_pdl(rope_kv_write_vec_kernel<float>, dim3(T), dim3(256), (size_t)rot * sizeof(float), stream, static_cast<float*>(qkv), inv_freq,
               inv_freq_lo, rot, pos_scale, tok_pos, tok_seq, block_table, bt_stride, static_cast<float*>(k_pool),
               static_cast<float*>(v_pool), nh, nkv, hd, page, write_kv);
  } else if (fast) {
    launch_pdl(rope_kv_write_vec_kernel<__nv_bfloat16>, dim3(T), dim3(256), (size_t)rot * sizeof(float), stream,
               static_cast<__nv_bfloat16*>(qkv), inv_freq, inv_freq_lo, rot, pos_scale, tok_pos, tok_seq, block_table, bt_stride,
               static_cast<__nv_bfloat16*>(k_pool), static_cast<__nv_bfloat16*>(v_pool), nh, nkv, hd, page, write_kv);
  } else {
    launch_pdl(rope_kv_write_kernel, dim3(T), dim3(256), 0, stream, qkv, dtype, inv_freq, inv_freq_lo, rot, pos_scale, tok_pos,
               tok_seq, block_table, bt_stride, k_pool, v_pool, nh, nkv, hd, page, write_kv);
  }
  return launch_status("rope_kv_write");
}
