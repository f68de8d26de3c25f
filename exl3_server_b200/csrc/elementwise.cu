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
__device__ inline void store_any(void* p, int dtype, int64_t i, float v) {
  if (dtype == DT_F32) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// h[t,:] = table[ids[t],:] * scale
__global__ void embed_kernel(const int* __restrict__ ids, const void* __restrict__ table,
                             int table_dtype, float* __restrict__ h, int H, int V, float scale) {
  const int t = blockIdx.x;
  const int id = ids[t];
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
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const void* __restrict__ y, int y_dtype,
                                   float y_scale, const void* __restrict__ w, int w_dtype, float eps,
                                   void* __restrict__ out, int out_dtype, float out_scale,
                                   const int* __restrict__ rows, int H) {
  __shared__ float red[32];
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* hr = h + (int64_t)r * H;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = hr[c];
    if (y) {
      v += load_any(y, y_dtype, (int64_t)r * H + c) * y_scale;
      hr[c] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = hr[c] * inv * load_any(w, w_dtype, c) * out_scale;   // same thread wrote hr[c]
    store_any(out, out_dtype, (int64_t)i * H + c, v);
  }
}

// out[t,i] = silu(gu[t,i]) * gu[t,I+i]
__global__ void silu_mul_kernel(const void* __restrict__ gu, void* __restrict__ out, int dtype,
                                int64_t total, int I) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t t = idx / I;
  const int i = (int)(idx - t * I);
  const float g = load_any(gu, dtype, t * 2 * I + i);
  const float u = load_any(gu, dtype, t * 2 * I + I + i);
  store_any(out, dtype, idx, g / (1.0f + expf(-g)) * u);
}

// One block per token.  qkv[t] = [q heads | k heads | v heads], each head_dim
// wide.  q and k are rotated in place (half-split pairs d, d + rot/2 with
// angle pos * pos_scale * inv_freq[d]); rotated k and plain v are written to
// the token's place in the paged cache.
__global__ void rope_kv_write_kernel(void* __restrict__ qkv, int dtype, const float* __restrict__ inv_freq,
                                     int rot, float pos_scale, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                     int bt_stride, void* __restrict__ k_pool, void* __restrict__ v_pool,
                                     int nh, int nkv, int hd, int page, int write_kv) {
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
  // rotated pairs of q and k
  const int n_rot_heads = nh + nkv;
  for (int i = threadIdx.x; i < n_rot_heads * half; i += blockDim.x) {
    const int head = i / half, d = i - head * half;
    float s, c;
    sincosf(p * inv_freq[d], &s, &c);
    const int64_t a = base + (int64_t)head * hd + d;
    const float x0 = load_any(qkv, dtype, a), x1 = load_any(qkv, dtype, a + half);
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
  if (!cache_ok) return;
  // features of k beyond the rotated ones pass through
  const int tail = hd - rot;
  for (int i = threadIdx.x; i < nkv * tail; i += blockDim.x) {
    const int g = i / tail, d = rot + (i - g * tail);
    store_any(k_pool, dtype, cache_base + (int64_t)g * page * hd + d,
              load_any(qkv, dtype, base + (int64_t)(nh + g) * hd + d));
  }
  for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x) {
    const int g = i / hd, d = i - g * hd;
    store_any(v_pool, dtype, cache_base + (int64_t)g * page * hd + d,
              load_any(qkv, dtype, base + (int64_t)(nh + nkv + g) * hd + d));
  }
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_embed(const int* ids, const void* table, int table_dtype, float* h, int T, int H,
                          int V, float scale, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H < 1 || V < 1) { set_error("embed: bad sizes T=%d H=%d V=%d", T, H, V); return ERR_BAD_ARGUMENT; }
  embed_kernel<<<T, 256, 0, stream>>>(ids, table, table_dtype, h, H, V, scale);
  return launch_status("embed");
}

extern "C" int exl3_add_rmsnorm(float* h, const void* y, int y_dtype, float y_scale, const void* w,
                                int w_dtype, float eps, void* out, int out_dtype, float out_scale,
                                const int* rows, int n_rows, int H, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  if (n_rows < 0 || H < 1) { set_error("add_rmsnorm: bad sizes rows=%d H=%d", n_rows, H); return ERR_BAD_ARGUMENT; }
  add_rmsnorm_kernel<<<n_rows, 256, 0, stream>>>(h, y, y_dtype, y_scale, w, w_dtype, eps, out, out_dtype,
                                                  out_scale, rows, H);
  return launch_status("add_rmsnorm");
}

extern "C" int exl3_silu_mul(const void* gu, void* out, int dtype, int T, int I, cudaStream_t stream) {
  const int64_t total = (int64_t)T * I;
  if (total == 0) return 0;
  if (T < 0 || I < 1) { set_error("silu_mul: bad sizes T=%d I=%d", T, I); return ERR_BAD_ARGUMENT; }
  const int64_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) { set_error("silu_mul: too many elements"); return ERR_UNSUPPORTED; }
  silu_mul_kernel<<<(unsigned)blocks, 256, 0, stream>>>(gu, out, dtype, total, I);
  return launch_status("silu_mul");
}

extern "C" int exl3_rope_kv_write(void* qkv, int dtype, const float* inv_freq, int rot, float pos_scale,
                                  const int* tok_pos, const int* tok_seq, const int* block_table,
                                  int bt_stride, void* k_pool, void* v_pool, int T, int nh, int nkv, int hd,
                                  int page, int write_kv, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || nh < 1 || nkv < 1 || hd < 2 || page < 1 || rot < 0 || rot > hd || (rot & 1)) {
    set_error("rope_kv_write: bad sizes T=%d heads=%d kv_heads=%d head_dim=%d rot=%d page=%d", T, nh, nkv,
              hd, rot, page);
    return ERR_BAD_ARGUMENT;
  }
  rope_kv_write_kernel<<<T, 256, 0, stream>>>(qkv, dtype, inv_freq, rot, pos_scale, tok_pos, tok_seq,
                                               block_table, bt_stride, k_pool, v_pool, nh, nkv, hd, page,
                                               write_kv);
  return launch_status("rope_kv_write");
}
