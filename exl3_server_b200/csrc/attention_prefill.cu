// Causal grouped-query attention of whole prompts over the paged cache, on the
// tensor cores (bfloat16 operands, float32 scores, softmax and accumulators).
//
// Same mathematics as attention_simt.cu (the reference's masked
// scaled-dot-product attention, src/model.cpp:539-548, 576-578), organised as a
// streaming softmax: a block owns 128 (heads of 64) or 64 (heads of 128)
// consecutive queries of one sequence and one head; each of its 4 warps owns
// 32 or 16 query rows.  It walks the sequence's
// key pages (64 keys per page) from the first page any of its queries may see
// to the page of its last query.  Per page: S = Q K^T with mma.m16n8k16, mask,
// running max / sum update in registers, O += P V.  K and V pages are copied
// to shared memory with cp.async, several pages ahead, in an XOR-swizzled layout
// that ldmatrix reads without bank conflicts.
//
// Requires head_dim 64 or 128 and a page size of 64; other shapes go through
// attention_simt.cu.
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace exl3 {

constexpr int PF_BQ = 64;       // queries per block of 4 warps
#ifndef PF_WARPS_64
#define PF_WARPS_64 4            // warps per block for heads of 64 (16 query rows each)
#endif
constexpr int PF_BK = 64;       // keys per step = page size

__device__ inline void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ inline void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ inline void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ inline void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ inline void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit; ex2.approx(-inf) = +0
__device__ inline float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ inline uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Element (row, col) of a [rows][HD] bfloat16 tile whose 16-byte chunks are
// XOR-swizzled with the row: returns the element offset of the chunk start.
template <int HD>
__device__ inline int swz(int row, int chunk) {
  return row * HD + ((chunk ^ (row & 7)) << 3);
}

// MT: 16-row tiles per warp; a block owns 64 * MT queries.  With MT = 2 every K
// and V fragment read from shared memory feeds two mma instructions.
template <int HD, int MT, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, HD == 64 ? 4 : 2)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_row_stride, __nv_bfloat16* __restrict__ out,
                    const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ row_start,
                    const int* __restrict__ row_pos0, const int* __restrict__ tile_seq,
                    const int* __restrict__ tile_q0, int nh, int nkv, int window, float scale_log2) {
  constexpr int BQ = 16 * MT * WARPS;
  constexpr int PF_THREADS = WARPS * 32;
  constexpr int CH = HD / 8;                         // 16-byte chunks per row
  constexpr int KS = HD / 16;                        // k16 steps over the head dimension
  constexpr int NB = PF_BK / 8;                      // n8 blocks of keys per page
  constexpr int DB = HD / 8;                         // n8 blocks of output features
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [BQ][HD]
  __nv_bfloat16* sK = sQ + BQ * HD;                                          // [STAGES][64][HD]
  __nv_bfloat16* sV = sK + STAGES * PF_BK * HD;                              // [STAGES][64][HD]

  // the caller lists the tiles with the most keys to visit first
  const int head = blockIdx.x, tile = blockIdx.y;   // blocks start in this order: all heads of tile 0, then tile 1, ...
  const int b = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = row_start[b + 1] - row_start[b];
  const int pos0 = row_pos0[b];
  const int g = head / (nh / nkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int rows = min(BQ, n_new - q0);              // valid queries in this tile
  const int p_first = pos0 + q0, p_last = pos0 + q0 + rows - 1;
  const int k_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  const int page_lo = k_lo / PF_BK, page_hi = p_last / PF_BK;
  const int* bt = block_table + (int64_t)b * bt_stride;

  // Q tile -> shared (rows past the end repeat the last valid row; they are never stored)
  const __nv_bfloat16* qbase = q + (int64_t)(row_start[b] + q0) * q_row_stride + (int64_t)head * HD;
  for (int c = tid; c < BQ * CH; c += PF_THREADS) {
    const int r = c / CH, ch = c - r * CH;
    cp_async16(sQ + swz<HD>(r, ch), qbase + (int64_t)min(r, rows - 1) * q_row_stride + ch * 8);
  }
  auto load_page = [&](int page_idx, int stage) {
    const int pg = bt[page_idx];
    const __nv_bfloat16* kp = k_pool + ((int64_t)pg * nkv + g) * PF_BK * HD;
    const __nv_bfloat16* vp = v_pool + ((int64_t)pg * nkv + g) * PF_BK * HD;
    __nv_bfloat16* dk = sK + stage * PF_BK * HD;
    __nv_bfloat16* dv = sV + stage * PF_BK * HD;
    for (int c = tid; c < PF_BK * CH; c += PF_THREADS) {
      const int r = c / CH, ch = c - r * CH;
      cp_async16(dk + swz<HD>(r, ch), kp + r * HD + ch * 8);
      cp_async16(dv + swz<HD>(r, ch), vp + r * HD + ch * 8);
    }
  };
  // STAGES - 1 pages are in flight ahead of the one being used
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (page_lo + st <= page_hi) load_page(page_lo + st, st);
    cp_async_commit();
  }

  uint32_t qf[MT][KS][4];
  float o[MT][DB][4];
  float m_run[MT][2], l_run[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int i = 0; i < DB; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[mt][i][j] = 0.0f;
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.0f;
  }
  const int wrow = warp * 16 * MT;                    // this warp's first row in the tile

  for (int pi = page_lo; pi <= page_hi; ++pi) {
    const int stage = (pi - page_lo) % STAGES;
    if (pi + STAGES - 1 <= page_hi) load_page(pi + STAGES - 1, (pi - page_lo + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    if (pi == page_lo) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
          ldmatrix_x4(qf[mt][ks], sQ + swz<HD>(wrow + mt * 16 + (lane & 15), ks * 2 + (lane >> 4)));
    }
    const __nv_bfloat16* tk = sK + stage * PF_BK * HD;
    const __nv_bfloat16* tv = sV + stage * PF_BK * HD;
    const int key0 = pi * PF_BK;
    // a warp whose rows all lie before this page has nothing to do here
    const bool warp_active = key0 <= p_first + wrow + 16 * MT - 1;
    if (warp_active) {
      // S = Q K^T for 16 * MT rows x 64 keys
      float s[MT][NB][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int j = 0; j < 4; ++j) s[mt][nb][j] = 0.0f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int nb2 = 0; nb2 < NB / 2; ++nb2) {
          uint32_t kb[4];
          const int krow = nb2 * 16 + (lane & 7) + ((lane >> 4) << 3);
          ldmatrix_x4(kb, tk + swz<HD>(krow, ks * 2 + ((lane >> 3) & 1)));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_16816(s[mt][nb2 * 2], qf[mt][ks], kb[0], kb[1]);
            mma_16816(s[mt][nb2 * 2 + 1], qf[mt][ks], kb[2], kb[3]);
          }
        }
      }
      // mask, running max and sum; the softmax scale is folded into the exponent:
      // p = 2^(s * scale_log2 - m), one multiply-add and one ex2 per score
      const bool need_mask = (key0 + PF_BK - 1 > p_first + wrow) || (window > 0 && key0 <= p_last - window);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int p_a = p_first + wrow + mt * 16 + gid, p_b = p_a + 8;
        if (need_mask) {                                  // selects, no branch per score
          const int lo_a = (window > 0) ? p_a - window : -1, lo_b = (window > 0) ? p_b - window : -1;
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int key = key0 + nb * 8 + tig * 2 + (j & 1);
              const int p = (j < 2) ? p_a : p_b, lo = (j < 2) ? lo_a : lo_b;
              const bool dead = (key > p) | (key <= lo);
              s[mt][nb][j] = dead ? -INFINITY : s[mt][nb][j];
            }
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float mx = -INFINITY;
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) mx = fmaxf(mx, fmaxf(s[mt][nb][2 * h], s[mt][nb][2 * h + 1]));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float mn = fmaxf(m_run[mt][h], mx * scale_log2);   // scale > 0: max and scale commute
          const float base = (mn == -INFINITY) ? 0.0f : mn;        // a row that has seen no key yet
          const float corr = fast_exp2(m_run[mt][h] - base);
          float sum = 0.0f;
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            const float p0 = fast_exp2(fmaf(s[mt][nb][2 * h], scale_log2, -base));
            const float p1 = fast_exp2(fmaf(s[mt][nb][2 * h + 1], scale_log2, -base));
            s[mt][nb][2 * h] = p0;
            s[mt][nb][2 * h + 1] = p1;
            sum += p0 + p1;
          }
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          l_run[mt][h] = l_run[mt][h] * corr + sum;
          m_run[mt][h] = mn;
          if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
            for (int db = 0; db < DB; ++db) {
              o[mt][db][2 * h] *= corr;
              o[mt][db][2 * h + 1] *= corr;
            }
          }
        }
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < PF_BK / 16; ++kk) {
        uint32_t pa[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          pa[mt][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
          pa[mt][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
          pa[mt][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
          pa[mt][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
        }
#pragma unroll
        for (int db2 = 0; db2 < DB / 2; ++db2) {
          uint32_t vb[4];
          const int vrow = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          ldmatrix_x4_trans(vb, tv + swz<HD>(vrow, db2 * 2 + (lane >> 4)));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_16816(o[mt][db2 * 2], pa[mt], vb[0], vb[1]);
            mma_16816(o[mt][db2 * 2 + 1], pa[mt], vb[2], vb[3]);
          }
        }
      }
    }
    __syncthreads();                                   // this stage is overwritten by the next load
  }

  // normalise and store
  __nv_bfloat16* obase = out + ((int64_t)(row_start[b] + q0) * nh + head) * HD;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int r_a = wrow + mt * 16 + gid, r_b = r_a + 8;
    const float inv_a = 1.0f / l_run[mt][0], inv_b = 1.0f / l_run[mt][1];
#pragma unroll
    for (int db = 0; db < DB; ++db) {
      const int d = db * 8 + tig * 2;
      if (r_a < rows)
        *reinterpret_cast<uint32_t*>(obase + (int64_t)r_a * nh * HD + d) =
            pack_bf16(o[mt][db][0] * inv_a, o[mt][db][1] * inv_a);
      if (r_b < rows)
        *reinterpret_cast<uint32_t*>(obase + (int64_t)r_b * nh * HD + d) =
            pack_bf16(o[mt][db][2] * inv_b, o[mt][db][3] * inv_b);
    }
  }
}

template <int HD, int MT, int STAGES, int WARPS>
static int launch_prefill(const void* q, int64_t q_row_stride, void* out, const void* k_pool, const void* v_pool,
                          const int* block_table, int bt_stride, const int* row_start, const int* row_pos0,
                          const int* tile_seq, const int* tile_q0, int n_tiles, int nh, int nkv, int window,
                          float scale, cudaStream_t stream) {
  const size_t smem = (size_t)(16 * MT * WARPS + 2 * STAGES * PF_BK) * HD * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD, MT, STAGES, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) { set_error("attn_prefill: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); return (int)e; }
    configured = true;
  }
  dim3 grid(nh, n_tiles);
  attn_prefill_kernel<HD, MT, STAGES, WARPS><<<grid, WARPS * 32, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(q), q_row_stride, static_cast<__nv_bfloat16*>(out),
      static_cast<const __nv_bfloat16*>(k_pool), static_cast<const __nv_bfloat16*>(v_pool), block_table,
      bt_stride, row_start, row_pos0, tile_seq, tile_q0, nh, nkv, window, scale * 1.4426950408889634f);
  return launch_status("attn_prefill");
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_attn_prefill_supported(int dtype, int hd, int page) {
  return dtype == DT_BF16 && (hd == 64 || hd == 128) && page == PF_BK;
}

// Queries per block for a head size: 128 for heads of 64, 64 for heads of 128.
extern "C" int exl3_attn_prefill_tile(int hd) { return hd == 64 ? 16 * PF_WARPS_64 : PF_BQ; }

// Tiles: tile i covers queries tile_q0[i] .. tile_q0[i] + tile - 1 (among the new
// tokens) of batch row tile_seq[i], with tile = exl3_attn_prefill_tile(hd).
extern "C" int exl3_attn_prefill(const void* q, int64_t q_row_stride, void* out, int dtype, const void* k_pool,
                                 const void* v_pool, const int* block_table, int bt_stride,
                                 const int* row_start, const int* row_pos0, const int* tile_seq,
                                 const int* tile_q0, int n_tiles, int nh, int nkv, int hd, int page, int window,
                                 float scale, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  if (!exl3_attn_prefill_supported(dtype, hd, page)) {
    set_error("attn_prefill: needs bfloat16, head_dim 64 or 128 and pages of 64, got type %d head_dim %d page %d",
              dtype, hd, page);
    return ERR_UNSUPPORTED;
  }
  if (n_tiles < 0 || nh < 1 || nkv < 1 || nh % nkv != 0 || n_tiles > 65535 || window < 0) {
    set_error("attn_prefill: bad sizes tiles=%d heads=%d kv_heads=%d window=%d", n_tiles, nh, nkv, window);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(q) || !aligned16(k_pool) || !aligned16(v_pool) || !aligned16(out) || q_row_stride % 8 != 0) {
    set_error("attn_prefill: q, k, v and out must be 16-byte aligned with a row stride in 16-byte units");
    return ERR_ALIGNMENT;
  }
  if (hd == 64)
    return launch_prefill<64, 1, 3, PF_WARPS_64>(q, q_row_stride, out, k_pool, v_pool, block_table, bt_stride, row_start, row_pos0,
                              tile_seq, tile_q0, n_tiles, nh, nkv, window, scale, stream);
  return launch_prefill<128, 1, 3, 4>(q, q_row_stride, out, k_pool, v_pool, block_table, bt_stride, row_start, row_pos0,
                             tile_seq, tile_q0, n_tiles, nh, nkv, window, scale, stream);
}
