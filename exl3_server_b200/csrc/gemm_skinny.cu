// Decode-shaped projection for batches of up to 128 rows on the 5th-generation tensor cores:
//   y[M,N] = x[M,K] . w[N,K]^T (+ bias), bfloat16 operands, float32 accumulation,
// with the weights as the 128-row operand of tcgen05.mma and the batch as its N (padded to 16): the weight matrix
// streams through shared memory exactly once for all rows, by TMA, and the accumulator [features x batch] sits in
// tensor memory.  The reference's counterparts are library matmuls (src/model.cpp:549-552, 558-560, 583-586).
//
// Work: a block owns R x 128 rows of w (R = 1 or 2: with two tiles a block reads its piece of x once for twice
// the weights).  A weight matrix of a few thousand rows has too few tiles for 148 SMs, so a tile's K range is cut
// over the S blocks of a thread-block cluster (S = 1 to 8, from N and K only).  Each block keeps its partial tile
// in its own shared memory; after a cluster barrier block r adds up, in block order, the partial values of batch
// rows r, r + S, ... through distributed shared memory and runs the epilogue for them.  No scratch in global
// memory, no atomics: a result depends on N, K and S only, never on M or on batch mates.
//
// Block of 6 warps: warp 0 issues the TMA copies (weights first, before griddepcontrol.wait: they do not depend
// on the kernel before this one; then the activations), warp 1 issues tcgen05.mma and owns the tensor memory,
// warps 2-5 are the epilogue (thread = feature).  Epilogues as in the weight-streaming GEMV (gemv_bf16.cuh):
// 0 plain, 1 silu(gate) * up over rows interleaved in eights, 2 into the residual with the pieces of the next
// norm (h += y * rho, x_raw = h * norm_w, sums of squares per 16 features), and optionally the consuming side of
// such a norm (results times rsqrt(sum of the producer's sums / width + eps) per batch row).
//
// Every wait on an mbarrier is bounded; a block that gives up records a code (exl3_gemm_skinny_status), skips its
// work, still joins both cluster barriers (every thread reaches them unconditionally) and frees its tensor
// memory.  TMA copies read this GPU's memory only and none is multicast.
#include "api.h"
#include "tcgen05.cuh"

#include <mutex>
#include <unordered_map>

namespace exl3 {

using namespace tc5;

constexpr int SK_BM = 128, SK_BK = 64, SK_UMMA_K = 16;
constexpr int SK_THREADS = 192;
constexpr int SK_MAX_ROWS = 128;
constexpr int SK_MAX_SPLIT = 8;
constexpr uint32_t SK_TILE_W = SK_BM * SK_BK * 2;      // one 128-row tile of a stage

static __device__ int g_sk_error = 0;

struct SkinnyArgs {
  void* y;
  const __nv_bfloat16* bias;
  int M, N, K;
  int MP;                        // M rounded up to 16: the instruction's N and the rows of an x tile
  int stages;
  int split;                     // blocks per cluster = cuts of K
  int rows_per;                  // batch rows a block finishes at most: ceil(MP / split)
  int tmem_cols;
  int out_f32;
  // epilogue 2, the producing side of a norm
  float* h;
  const void* norm_w;
  __nv_bfloat16* x_raw;
  float* ss_out;                 // [M, ceil(N / 16)]
  float rho;
  int norm_w_f32;
  // the consuming side
  const float* ss_in;            // [>= M, ss_blocks]
  int ss_blocks;
  float eps, width;
};

__device__ inline uint32_t sk_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ inline void sk_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ inline void sk_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ inline void sk_cluster_sync() { sk_cluster_arrive(); sk_cluster_wait(); }
// Arrives only once `loaded` is in its register: the loads it was computed from have come back by then.
__device__ inline void sk_cluster_arrive_after(float loaded) {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::"f"(loaded) : "memory");
}
// The address of this block's shared-memory location `addr` in the block of rank `rank` of the cluster.
__device__ inline uint32_t sk_map_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ inline float4 sk_ld_cluster4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// R: 128-row tiles of w per block.
template <int EPI, bool SCALE, int R>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const SkinnyArgs a) {
  extern __shared__ unsigned char sk_smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(sk_smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr uint32_t STAGE_W = R * SK_TILE_W;
  constexpr int RW = R * SK_BM;                              // features of a block
  const uint32_t stage_x = (uint32_t)a.MP * SK_BK * 2;
  const int S = a.split;
  unsigned char* sW = base;
  unsigned char* sX = base + (size_t)a.stages * STAGE_W;
  float* part = reinterpret_cast<float*>(base);          // [MP][RW]: takes the ring's place when the ring is done with
  uint64_t* full = reinterpret_cast<uint64_t*>(sX + (size_t)a.stages * stage_x);   // [stages] copies landed
  uint64_t* empty = full + a.stages;                      // [stages] the MMAs that read the stage are done
  uint64_t* acc_full = empty + a.stages;                  // the accumulator is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  float* s_inv = reinterpret_cast<float*>(tmem_slot + 2); // [rows_per] SCALE: factor of the i-th batch row of this block

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)sk_cluster_rank();
  const int tile = blockIdx.x / S;
  const int n0 = tile * RW;
  const int ksteps = (a.K + SK_BK - 1) / SK_BK;
  const int ks0 = (int)((int64_t)ksteps * rank / S), ks1 = (int)((int64_t)ksteps * (rank + 1) / S);
  const int nk = ks1 - ks0;
  const int pre = nk < a.stages ? nk : a.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    mbar_init(acc_full, 1);
    mbar_init_fence();
    // the first weights are asked for at once: they need nothing but this thread's own barriers
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(full + i, STAGE_W + stage_x);
      tma_load_2d(sW + (size_t)i * STAGE_W, &map_w, full + i, (ks0 + i) * SK_BK, n0);
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(a.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 0) {
    // ---- producer ---------------------------------------------------------------------------------------
    pdl_wait();                                           // x is the previous kernel's output
    if (lane == 0)
      for (int i = 0; i < pre; ++i) tma_load_2d(sX + (size_t)i * stage_x, &map_x, full + i, (ks0 + i) * SK_BK, 0);
    __syncwarp();
    int issued = pre;
    // the ring's stage and round of step i, counted along (a division by the run-time stage count in every step
    // is part of what the one issuing thread pays per step)
    int s = pre % a.stages, round = pre / a.stages;
    for (int i = pre; i < nk; ++i) {
      if (!mbar_wait(empty + s, (round & 1) ^ 1)) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(full + s, STAGE_W + stage_x);
        tma_load_2d(sW + (size_t)s * STAGE_W, &map_w, full + s, (ks0 + i) * SK_BK, n0);
        tma_load_2d(sX + (size_t)s * stage_x, &map_x, full + s, (ks0 + i) * SK_BK, 0);
      }
      __syncwarp();
      issued = i + 1;
      if (++s == a.stages) { s = 0; ++round; }
    }
    if (!ok) {
      if (lane == 0) atomicExch(&g_sk_error, 1);
      // copies still in flight must land before the block's shared memory goes away
      for (int back = 1; back <= a.stages && back <= issued; ++back) {
        const int j = issued - back;
        mbar_wait(full + (j % a.stages), (j / a.stages) & 1);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ---------------------------------------------------------------------------------------
    const uint32_t idesc = idesc_bf16(SK_BM, a.MP);
    int s = 0, round = 0;
    for (int i = 0; i < nk; ++i) {
      if (!mbar_wait(full + s, round & 1)) { ok = false; break; }
      fence_after();
      if (lane == 0) {
        const uint64_t db = smem_desc_k128(smem_u32(sX + (size_t)s * stage_x));
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint64_t da = smem_desc_k128(smem_u32(sW + (size_t)s * STAGE_W + r * SK_TILE_W));
#pragma unroll
          for (int k = 0; k < SK_BK / SK_UMMA_K; ++k)
            mma_ss(tmem_base + (uint32_t)(r * a.MP), da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(empty + s);
      }
      __syncwarp();
      if (++s == a.stages) { s = 0; ++round; }
    }
    if (ok) {
      if (lane == 0) mma_commit(acc_full);
      __syncwarp();
    } else if (lane == 0) {
      atomicExch(&g_sk_error, 2);
    }
  } else {
    // ---- epilogue, first half: this block's partial tile into its shared memory ---------------------------
    const int q = warp & 3;                                // the 32 tensor-memory lanes this warp may read
    const int t = q * 32 + lane;
    pdl_wait();
    if (SCALE) {
      // the factors of the batch rows this block will finish: sums of the producer's sums, in a fixed order
      for (int i = q; rank + i * S < a.M; i += 4) {
        const int m = rank + i * S;
        float ss = 0.0f;
        for (int p = lane; p < a.ss_blocks; p += 32) ss += __ldcg(a.ss_in + (int64_t)m * a.ss_blocks + p);
        ss = warp_sum(ss);
        if (lane == 0) s_inv[i] = 1.0f / sqrtf(ss / a.width + a.eps);
      }
    }
    ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0));   // the same for the whole warp: shuffles follow
    if (!ok && lane == 0) atomicExch(&g_sk_error, 3);
    fence_after();
    if (ok) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(r * a.MP);
        for (int c = 0; c < a.MP; c += 16) {
          uint32_t v[16];
          tmem_ld16(taddr + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(c + j) * RW + r * SK_BM + t] = __uint_as_float(v[j]);
        }
      }
    }
    fence_before();
  }

  // every block of the cluster has its partial tile in place (or has given up: then its values are not used,
  // because the error code makes the host reject the step)
  sk_cluster_sync();

  // The second cluster barrier keeps a block alive while others may still read its shared memory.  A warp arrives
  // as soon as its own last loads from other blocks have come back, and waits only at the very end, so that the
  // barrier's trip overlaps the arithmetic and the stores.
  bool arrived = false;
  if (warp < 2 || !ok) { sk_cluster_arrive(); arrived = true; }

  if (warp >= 2 && ok) {
    // ---- epilogue, second half: batch rows rank, rank + S, ... of the whole tile ----------------------------
    // A warp takes a batch row at a time, a lane four neighbouring features of it: 16-byte loads from the other
    // blocks' shared memory (the path between SMs is slow in small pieces) and 8- or 16-byte stores.
    const int q = warp & 3;
    const int ss_out_blocks = (a.N + 15) >> 4;
    const bool vec = (a.N & 3) == 0;                        // rows of y, h and x_raw start on 16-byte boundaries
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int f0 = r * SK_BM + 4 * lane;
      const int n = n0 + f0;
      uint32_t peer[SK_MAX_SPLIT];
#pragma unroll
      for (int j = 0; j < SK_MAX_SPLIT; ++j) peer[j] = j < S ? sk_map_rank(smem_u32(part + f0), (uint32_t)j) : 0u;
      float bias_v[4] = {0.0f, 0.0f, 0.0f, 0.0f}, wn[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (n + e < a.N) {
          if (a.bias) bias_v[e] = __bfloat162float(a.bias[n + e]);
          if (EPI == 2)
            wn[e] = a.norm_w_f32 ? __ldg(static_cast<const float*>(a.norm_w) + n + e)
                                 : __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(a.norm_w) + n + e));
        }
      }
      // the loads of up to ROWS batch rows are in flight together: a trip to another SM's shared memory takes about
      // a microsecond, whatever it carries
      constexpr int ROWS = 3;
      for (int i0 = q; rank + i0 * S < a.M; i0 += 4 * ROWS) {
        float4 vv[ROWS][SK_MAX_SPLIT];
        float h_all[ROWS][4];
#pragma unroll
        for (int u = 0; u < ROWS; ++u) {
          const int m = rank + (i0 + 4 * u) * S;
          const bool row = m < a.M;
#pragma unroll
          for (int j = 0; j < SK_MAX_SPLIT; ++j)
            vv[u][j] = (j < S && row) ? sk_ld_cluster4(peer[j] + (uint32_t)m * RW * 4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
          for (int e = 0; e < 4; ++e) h_all[u][e] = 0.0f;
          if (EPI == 2 && row) {
            if (vec) {
              if (n < a.N) {
                const float4 hv = __ldcg(reinterpret_cast<const float4*>(a.h + (int64_t)m * a.N + n));
                h_all[u][0] = hv.x; h_all[u][1] = hv.y; h_all[u][2] = hv.z; h_all[u][3] = hv.w;
              }
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) if (n + e < a.N) h_all[u][e] = __ldcg(a.h + (int64_t)m * a.N + n + e);
            }
          }
        }
        if (r == R - 1 && rank + (i0 + 4 * ROWS) * S >= a.M) {     // this warp's last loads
          float got = 0.0f;
#pragma unroll
          for (int u = 0; u < ROWS; ++u)
#pragma unroll
            for (int j = 0; j < SK_MAX_SPLIT; ++j) got += vv[u][j].x + vv[u][j].y + vv[u][j].z + vv[u][j].w;
          sk_cluster_arrive_after(got);
          arrived = true;
        }
#pragma unroll
        for (int u = 0; u < ROWS; ++u) {
        const int i = i0 + 4 * u;
        const int m = rank + i * S;
        if (m >= a.M) break;                               // the same for every lane of the warp
        const float4* v = vv[u];
        const float* h_old = h_all[u];
        float s[4] = {v[0].x, v[0].y, v[0].z, v[0].w};
#pragma unroll
        for (int j = 1; j < SK_MAX_SPLIT; ++j) {            // block order; the zeros of absent blocks change nothing
          s[0] += v[j].x; s[1] += v[j].y; s[2] += v[j].z; s[3] += v[j].w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (SCALE) s[e] *= s_inv[i];
          s[e] += bias_v[e];
        }
        if (EPI == 0) {
          if (a.out_f32) {
            float* dst = static_cast<float*>(a.y) + (int64_t)m * a.N + n;
            if (vec) { if (n < a.N) *reinterpret_cast<float4*>(dst) = make_float4(s[0], s[1], s[2], s[3]); }
            else {
#pragma unroll
              for (int e = 0; e < 4; ++e) if (n + e < a.N) dst[e] = s[e];
            }
          } else {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.y) + (int64_t)m * a.N + n;
            if (vec) {
              if (n < a.N) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(s[0], s[1]), hi = __floats2bfloat162_rn(s[2], s[3]);
                *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
              }
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) if (n + e < a.N) dst[e] = __float2bfloat16_rn(s[e]);
            }
          }
        } else if (EPI == 1) {
          // rows in eights: of every four lanes the first two hold gate rows, the other two the up rows of the same
          // features (N is a multiple of 16 here)
          float o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float up = __shfl_down_sync(0xffffffffu, s[e], 2);
            o[e] = s[e] / (1.0f + expf(-s[e])) * up;
          }
          if ((lane & 2) == 0 && n < a.N) {
            const int f = ((n >> 4) << 3) + (n & 7);
            if (a.out_f32) {
              *reinterpret_cast<float4*>(static_cast<float*>(a.y) + (int64_t)m * (a.N >> 1) + f) = make_float4(o[0], o[1], o[2], o[3]);
            } else {
              const __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
              *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(a.y) + (int64_t)m * (a.N >> 1) + f) =
                  make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
            }
          }
        } else {
          float hv[4], sq = 0.0f;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // the output is rounded to bfloat16 as it would be on its way through memory
            hv[e] = h_old[e] + __bfloat162float(__float2bfloat16_rn(s[e])) * a.rho;
            if (n + e < a.N) sq += hv[e] * hv[e];
          }
          float* hp = a.h + (int64_t)m * a.N + n;
          __nv_bfloat16* xp = a.x_raw + (int64_t)m * a.N + n;
          if (vec) {
            if (n < a.N) {
              *reinterpret_cast<float4*>(hp) = make_float4(hv[0], hv[1], hv[2], hv[3]);
              const __nv_bfloat162 lo = __floats2bfloat162_rn(hv[0] * wn[0], hv[1] * wn[1]);
              const __nv_bfloat162 hi = __floats2bfloat162_rn(hv[2] * wn[2], hv[3] * wn[3]);
              *reinterpret_cast<uint2*>(xp) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
            }
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (n + e < a.N) { hp[e] = hv[e]; xp[e] = __float2bfloat16_rn(hv[e] * wn[e]); }
          }
          sq += __shfl_xor_sync(0xffffffffu, sq, 1);
          sq += __shfl_xor_sync(0xffffffffu, sq, 2);
          if ((lane & 3) == 0 && n < a.N) a.ss_out[(int64_t)m * ss_out_blocks + (n >> 4)] = sq;
        }
        }
      }
    }
  }

  if (!arrived) sk_cluster_arrive();
  sk_cluster_wait();
  fence_after();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(a.tmem_cols) : "memory");
}

// ---- host side ---------------------------------------------------------------------------------------------

static int sk_sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

// Tensor maps are pure functions of (address, rows, K, box): kept, so that a step replayed eagerly does not encode
// them again.  Weights come back with the same address for ever; activations with a handful of addresses.
struct SkMapKey {
  const void* p; int64_t rows; int K; int box;
  bool operator==(const SkMapKey& o) const { return p == o.p && rows == o.rows && K == o.K && box == o.box; }
};
struct SkMapHash {
  size_t operator()(const SkMapKey& k) const {
    return std::hash<const void*>()(k.p) ^ (std::hash<int64_t>()(k.rows) * 31) ^ (std::hash<int>()(k.K) * 131) ^ (size_t)k.box;
  }
};
static int sk_map(CUtensorMap* out, const void* p, int64_t rows, int K, int box) {
  static std::mutex mu;
  static std::unordered_map<SkMapKey, CUtensorMap, SkMapHash> cache;
  std::lock_guard<std::mutex> lock(mu);
  const SkMapKey key{p, rows, K, box};
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  const int rc = make_map_k64(out, p, rows, K, box, "gemm_skinny");
  if (rc) return rc;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

// Cuts of K for a weight matrix [N, K]: as many as still let all blocks run at once, two to an SM (a second wave
// costs its full length), at most 8 and at least two 64-wide steps per block.  Measured at 2304 x 2304 ... 11520 x
// 2304 with 8 and 64 rows: 5 cuts for 54 tiles, 3 for 90, 8 for 18.  From N and K only, so that a result never
// depends on the batch.
// Clusters of s blocks that run at once with two blocks to an SM, as the driver counts them for this kernel's
// block (192 threads, some 100 KB of shared memory).  A cluster's blocks must find their SMs in one of the GPU's
// parts, and the parts are not equal: on the B200 measured, 296 / 148 / 93 / 71 / 56 / 45 / 37 / 33 clusters of 1
// to 8 (a kernel whose blocks wait 20 us takes 20 us up to these counts and 40 us from one more: the same numbers).
// One cluster too many costs a second round of its full length: 6144 x 4096 in 6 cuts (48 clusters) 15.6 us, in 5
// cuts 10.7 us; 4608 x 4096 in 8 cuts 12.9 us, in 7 cuts 8.8 us.  From the device only: the answer must not depend
// on the batch, or a row's result would depend on its batch.
// never launched: a block of this kernel's shape for the driver's count
__global__ void __launch_bounds__(SK_THREADS) sk_block_shape_kernel() {}

static int sk_max_clusters(int s) {
  static int cache[SK_MAX_SPLIT + 1] = {};
  if (s < 1 || s > SK_MAX_SPLIT) return 0;
  if (cache[s] == 0) {
    int n = 0;
    const int smem = 100 * 1024;
    cudaError_t e = cudaFuncSetAttribute(sk_block_shape_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)(8 * s));
      cfg.blockDim = dim3(SK_THREADS);
      cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = (unsigned)s;
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      cfg.attrs = at;
      cfg.numAttrs = 1;
      e = cudaOccupancyMaxActiveClusters(&n, sk_block_shape_kernel, &cfg);
    }
    if (e != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = 8 * ((2 * (sk_sm_count() / 8)) / s);             // eight equal parts: a little too many for some s
      if (n < 1) n = 1;
    }
    cache[s] = n;
  }
  return cache[s];
}

static int sk_auto_split(int N, int K) {
  const int n_tiles = ceil_div(N, SK_BM), ksteps = ceil_div(K, SK_BK);
  int s = 2 * sk_sm_count() / n_tiles;
  if (s > SK_MAX_SPLIT) s = SK_MAX_SPLIT;
  while (s > 1 && ksteps / s < 2) --s;
  // fewer cuts when the tiles' clusters would not all run at once (a second round of clusters costs its full length)
  while (s > 1 && n_tiles > sk_max_clusters(s)) --s;
  if (s < 1) s = 1;
  // More tiles than SMs, and no cut: the cuts that pairs of tiles would get when a block takes two (as it does
  // for few rows, below): 32768 x 4096 at 1 to 32 rows 42.9-46.2 us with two tiles a block and two cuts against
  // 45.3-48.2 us with one and none; at 48 and 64 rows, a tile a block, the two cuts cost 1 us of 50.
  if (s == 1 && n_tiles > sk_sm_count()) {
    const int pairs = ceil_div(n_tiles, 2);
    int s2 = 2 * sk_sm_count() / pairs;
    if (s2 > SK_MAX_SPLIT) s2 = SK_MAX_SPLIT;
    while (s2 > 1 && (ksteps / s2 < 2 || pairs > sk_max_clusters(s2))) --s2;
    if (s2 >= 2) s = s2;
  }
  return s;
}

// Two tiles per block (the block's piece of x is then read once for twice the weights) where there are more
// tiles than SMs and the blocks of two tiles still fill the GPU one and a half times, for up to 32 rows (an
// output head of 122753 x 2304: 87.8 / 90.5 / 93.3 / 97.7 us at 1 / 8 / 16 / 32 rows against 95.1 / 97.5 / 100.5 /
// 105.1 with a tile a block, but 132.6 against 114.2 at 64 rows); for more rows only with many times more tiles
// than SMs.  Changes no result (the cuts of K stay what N and K say).
static int sk_auto_tiles(int N, int split, int M) {
  const int n_tiles = ceil_div(N, SK_BM), sms = sk_sm_count();
  if (M <= 32) return n_tiles > sms && 2 * ceil_div(n_tiles, 2) * split >= 3 * sms ? 2 : 1;
  return n_tiles * split >= 8 * sms ? 2 : 1;
}

template <int EPI, bool SCALE, int R>
static int sk_launch(const CUtensorMap& mw, const CUtensorMap& mx, const SkinnyArgs& a, int n_blocks, size_t smem,
                     cudaStream_t stream) {
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<EPI, SCALE, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_error("gemm_skinny: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); return (int)e; }
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)n_blocks);
  cfg.blockDim = dim3(SK_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)a.split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<EPI, SCALE, R>, mw, mx, a);
  return launch_status("gemm_skinny");
}

}  // namespace exl3

using namespace exl3;

// 0 when no block has given up on a wait since the last call; else 1 (copies), 2 (MMA), 3 (accumulator).
extern "C" int exl3_gemm_skinny_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_sk_error, sizeof(int));
  if (v) { int z = 0; cudaMemcpyToSymbol(g_sk_error, &z, sizeof(int)); }
  return v;
}

extern "C" int exl3_gemm_skinny_max_rows() { return SK_MAX_ROWS; }

// Clusters of s blocks that run at once (two blocks an SM): what the choice of cuts rests on.
extern "C" int exl3_gemm_skinny_max_clusters(int s) { return sk_max_clusters(s); }

// The split that split = 0 chooses for a weight matrix [N, K].
extern "C" int exl3_gemm_skinny_split(int N, int K) { return sk_auto_split(N, K); }

// Arguments as exl3_gemv_bf16_normed, for 1 <= M <= 128 rows; ss_in and ss_out are [rows, blocks] with M rows at
// least.  split: blocks that share a tile's K range (1 to 8), 0: chosen from N and K.  tiles: 128-row tiles per
// block (1 or 2), 0: chosen.
extern "C" int exl3_gemm_skinny(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N,
                                int K, int epilogue, const float* ss_in, int ss_blocks, float eps, float width,
                                float* h, float rho, const void* norm_w, int norm_w_dtype, void* x_raw,
                                float* ss_out, int split, int tiles, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > SK_MAX_ROWS || N < 0 || K < 8 || K % 8 != 0 || epilogue < 0 || epilogue > 2 ||
      (epilogue == 1 && N % 16 != 0) || (ss_in != nullptr && (ss_blocks < 1 || !(width > 0.0f))) ||
      split < 0 || split > SK_MAX_SPLIT || tiles < 0 || tiles > 2) {
    set_error("gemm_skinny: needs 1 <= M <= %d, K a multiple of 8, N a multiple of 16 when gated, split 0 to %d, tiles "
              "0 to 2; got M=%d N=%d K=%d epilogue=%d split=%d tiles=%d", SK_MAX_ROWS, SK_MAX_SPLIT, M, N, K, epilogue,
              split, tiles);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(x) || !aligned16(w)) { set_error("gemm_skinny: x and w must be 16-byte aligned"); return ERR_ALIGNMENT; }
  SkinnyArgs a = {};
  if (epilogue == 2) {
    if (!h || !norm_w || !x_raw || !ss_out || (norm_w_dtype != DT_F32 && norm_w_dtype != DT_BF16)) {
      set_error("gemm_skinny: the residual epilogue needs h, a float32 or bfloat16 norm weight, x_raw and ss_out");
      return ERR_BAD_ARGUMENT;
    }
    a.h = h;
    a.norm_w = norm_w;
    a.x_raw = static_cast<__nv_bfloat16*>(x_raw);
    a.ss_out = ss_out;
    a.rho = rho;
    a.norm_w_f32 = norm_w_dtype == DT_F32;
  } else if (out_dtype != DT_F32 && out_dtype != DT_BF16) {
    set_error("gemm_skinny: unsupported output type %d", out_dtype);
    return ERR_UNSUPPORTED;
  }
  a.y = y;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.M = M; a.N = N; a.K = K;
  a.MP = (M + 15) / 16 * 16;
  a.out_f32 = out_dtype == DT_F32;
  a.ss_in = ss_in; a.ss_blocks = ss_blocks; a.eps = eps; a.width = width;
  const int ksteps = ceil_div(K, SK_BK);
  a.split = split > 0 ? split : sk_auto_split(N, K);
  if (a.split > ksteps) a.split = ksteps;
  const int R = tiles > 0 ? tiles : sk_auto_tiles(N, a.split, M);
  a.rows_per = ceil_div(a.MP, a.split);
  const int cols = R * a.MP;
  a.tmem_cols = cols <= 32 ? 32 : (cols <= 64 ? 64 : (cols <= 128 ? 128 : 256));
  // shared memory: the ring; the partial tile [MP][R * 128] floats takes its place afterwards and must fit it.
  // As many stages as a block has steps, at most 4; fewer when two blocks can share an SM that way.
  const size_t stage = (size_t)R * SK_TILE_W + (size_t)a.MP * SK_BK * 2;
  const size_t part = (size_t)a.MP * R * SK_BM * 4;
  const size_t fixed = 1024 /* alignment */ + (size_t)(2 * 4 + 1) * 8 + 16 + (size_t)a.rows_per * 4 + 64;
  const int per_block = ceil_div(ksteps, a.split);
  int stages = per_block < 4 ? per_block : 4;
  if (stages == 4 && fixed + 3 * stage <= 113 * 1024 && fixed + 4 * stage > 113 * 1024) stages = 3;
  while ((size_t)stages * stage < part) ++stages;
  a.stages = stages;
  const size_t smem = fixed + (size_t)stages * stage;
  if (smem > 227 * 1024) { set_error("gemm_skinny: %zu bytes of shared memory needed", smem); return ERR_UNSUPPORTED; }
  CUtensorMap mw, mx;
  int rc = sk_map(&mw, w, N, K, R * SK_BM);
  if (rc) return rc;
  rc = sk_map(&mx, x, M, K, a.MP);
  if (rc) return rc;
  const int n_blocks = ceil_div(N, R * SK_BM) * a.split;
  const bool scale = ss_in != nullptr;
#define EXL3_SK2(EPI, R_) return scale ? sk_launch<EPI, true, R_>(mw, mx, a, n_blocks, smem, stream) \
                                       : sk_launch<EPI, false, R_>(mw, mx, a, n_blocks, smem, stream)
#define EXL3_SK(EPI) if (R == 1) { EXL3_SK2(EPI, 1); } else { EXL3_SK2(EPI, 2); }
  if (epilogue == 0) { EXL3_SK(0) }
  if (epilogue == 1) { EXL3_SK(1) }
  EXL3_SK(2)
#undef EXL3_SK
#undef EXL3_SK2
}
