// Sampling with filters on the device: the reference's sampler (sample_token,
// src/model.cpp:667-757) step for step, one block per row of logits.
//
//   penalties over the context (a kernel of its own, below), then
//   the 2048 largest logits in descending order (ties: the smaller index first),
//   p[i] = exp(logit[i] / T - max) as float32, sums in float64,
//   min-p: cut before the first candidate whose share is below min_p * the largest share,
//   top-k: at most k candidates,
//   top-p: cut after the first candidate at which the running share reaches top_p,
//   and the token at which the running sum of what is kept reaches u * its total.
//
// Only the chosen ids cross to the host; with the sampler on the host a step
// carries the whole rows there (vocabulary x 4 bytes each) and sorts them.
//
// The candidates are found without sorting the vocabulary: a radix select over
// the float bits (four passes of 256 bins over the row, which stays in L2)
// gives the 2048th largest value; when several tokens share that value the
// select goes on over their indices, so exactly 2048 tokens pass.  They are
// sorted in shared memory (bitonic, 64-bit keys: value bits above, inverted
// index below, all different).
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace exl3 {

constexpr int SF_THREADS = 1024;
constexpr int SF_CAP = 2048;                     // candidates: max(top_k, 2048) in the reference; top_k above it is refused here

// float bits -> unsigned keys in the floats' order
__device__ inline uint32_t sf_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ inline float sf_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct SfRow {            // one row's options, as the host gives them (float64 [R, 5])
  double temperature, top_k, top_p, min_p, u;
};

__global__ void __launch_bounds__(SF_THREADS)
sample_filtered_kernel(const float* __restrict__ logits, const SfRow* __restrict__ rows, int* __restrict__ out, int V) {
  // cand and acc hold nothing while the select runs: its histograms, one per warp, lie in their place.  (Logits
  // crowd into a few bins of the leading byte, and additions to one address of shared memory go one after the
  // other; a histogram per warp keeps the warps apart.  Measured, it made no difference to the kernel's time: the
  // passes over the row through one SM's memory pipe are what it costs.)
  __shared__ __align__(16) unsigned char raw[SF_CAP * 16];
  unsigned long long* cand = reinterpret_cast<unsigned long long*>(raw);       // (key << 32) | ~index, sorted descending
  double* acc = reinterpret_cast<double*>(raw + SF_CAP * 8);                   // running sums of probs
  unsigned (*whist)[256] = reinterpret_cast<unsigned (*)[256]>(raw);           // [warps][256]
  static_assert(sizeof(unsigned) * 256 * (SF_THREADS / 32) <= sizeof(raw), "the warps' histograms fit");
  __shared__ float probs[SF_CAP];
  __shared__ unsigned hist[256];
  __shared__ double warp_tot[SF_THREADS / 32];
  __shared__ unsigned long long sel_prefix;
  __shared__ unsigned sel_remaining, n_cand, same;
  __shared__ int first_below, first_hit, first_draw;
  const float* row = logits + (int64_t)blockIdx.x * V;
  const SfRow o = rows[blockIdx.x];
  const int tid = threadIdx.x;
  const int M = V < SF_CAP ? V : SF_CAP;

  // Every token's (value, inverted index) key.  One block reads its whole row several times over and an SM has
  // only so many loads on their way: 16-byte loads, four of a thread at a time, make a pass a few round trips
  // to L2 (rows start at any multiple of 4 bytes: the pieces before and after the aligned part go one by one).
  auto key_of = [&](float v, int i) { return ((unsigned long long)sf_key(v) << 32) | (unsigned)(~(unsigned)i); };
  const int head = min(V, (int)((4 - ((reinterpret_cast<uintptr_t>(row) >> 2) & 3)) & 3));
  const int n_vec = (V - head) / 4;
  const float4* row4 = reinterpret_cast<const float4*>(row + head);
  auto for_each = [&](auto&& f) {
    constexpr int AHEAD = 4;
    for (int i = tid; i < head; i += SF_THREADS) f(key_of(row[i], i));
    for (int j0 = tid; j0 < n_vec; j0 += SF_THREADS * AHEAD) {
      float4 v[AHEAD];
#pragma unroll
      for (int a = 0; a < AHEAD; ++a) {
        const int j = j0 + a * SF_THREADS;
        v[a] = j < n_vec ? row4[j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
#pragma unroll
      for (int a = 0; a < AHEAD; ++a) {
        const int j = j0 + a * SF_THREADS;
        if (j < n_vec) {
          const int i = head + 4 * j;
          f(key_of(v[a].x, i));
          f(key_of(v[a].y, i + 1));
          f(key_of(v[a].z, i + 2));
          f(key_of(v[a].w, i + 3));
        }
      }
    }
    for (int i = head + 4 * n_vec + tid; i < V; i += SF_THREADS) f(key_of(row[i], i));
  };

  // ---- the M largest (value, then smaller index): radix select on the composite key -------------
  unsigned long long thresh = 0;                 // everything passes when the row is no longer than the cap
  if (V > SF_CAP) {
    if (tid == 0) { sel_prefix = 0; sel_remaining = (unsigned)M; }
    __syncthreads();
    // the value's four bytes; the index's four only when tokens with the threshold's value are too many
    for (int shift = 56; shift >= 0; shift -= 8) {
      for (int b = tid; b < 256 * (SF_THREADS / 32); b += SF_THREADS) whist[0][b] = 0;
      __syncthreads();
      const unsigned long long prefix = sel_prefix;
      const unsigned long long mask = shift == 56 ? 0ull : (~0ull << (shift + 8));
      for_each([&](unsigned long long c) {
        if ((c & mask) == prefix) atomicAdd(&whist[tid >> 5][(unsigned)(c >> shift) & 255u], 1u);
      });
      __syncthreads();
      if (tid < 256) {
        unsigned n = 0;
        for (int w = 0; w < SF_THREADS / 32; ++w) n += whist[w][tid];
        hist[tid] = n;
      }
      __syncthreads();
      if (tid == 0) {
        unsigned cum = 0, rem = sel_remaining;
        int digit = 0;
        for (int b = 255; b >= 0; --b) {
          if (cum + hist[b] >= rem) { digit = b; break; }
          cum += hist[b];
        }
        sel_remaining = rem - cum;               // how many of this digit's tokens still pass
        sel_prefix = prefix | ((unsigned long long)digit << shift);
        same = hist[digit];                      // after the value's last byte: the tokens with the threshold's value
      }
      __syncthreads();
      // if all tokens with this value pass, their indices need no select: the threshold is (value, any index)
      if (shift == 32 && same == sel_remaining) break;
    }
    thresh = sel_prefix;
  }
  if (tid == 0) n_cand = 0;
  for (int i = tid; i < SF_CAP; i += SF_THREADS) cand[i] = 0ull;   // padding sorts last
  __syncthreads();
  for_each([&](unsigned long long c) {
    if (c >= thresh) {
      const unsigned at = atomicAdd(&n_cand, 1u);
      if (at < (unsigned)SF_CAP) cand[at] = c;
    }
  });
  __syncthreads();

  // ---- sorted descending: bitonic over the 2048 slots --------------------------------------------
  for (int k = 2; k <= SF_CAP; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < SF_CAP; i += SF_THREADS) {
        const int l = i ^ j;
        if (l > i) {
          const unsigned long long a = cand[i], b = cand[l];
          const bool desc = (i & k) == 0;
          if (desc ? a < b : a > b) { cand[i] = b; cand[l] = a; }
        }
      }
      __syncthreads();
    }
  }
  auto token_of = [&](int i) { return (int)(~(unsigned)(cand[i] & 0xffffffffull)); };
  if (!(o.temperature > 0.0)) {                  // greedy: the first maximum
    if (tid == 0) out[blockIdx.x] = token_of(0);
    return;
  }

  // ---- probabilities as the reference rounds them, their running sums in float64 ------------------
  const float inv_t = __fdiv_rn(1.0f, (float)o.temperature);
  const float maxl = __fmul_rn(sf_value((uint32_t)(cand[0] >> 32)), inv_t);
  for (int i = tid; i < SF_CAP; i += SF_THREADS)
    probs[i] = i < M ? expf(__fsub_rn(__fmul_rn(sf_value((uint32_t)(cand[i] >> 32)), inv_t), maxl)) : 0.0f;
  __syncthreads();
  {
    // inclusive scan: two neighbours per thread, then warps, then the warps' totals
    const int i0 = 2 * tid;
    const double a0 = (double)probs[i0], a1 = a0 + (double)probs[i0 + 1];
    double run = a1;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const double v = __shfl_up_sync(0xffffffffu, run, s);
      if ((tid & 31) >= s) run += v;
    }
    if ((tid & 31) == 31) warp_tot[tid >> 5] = run;
    __syncthreads();
    if (tid < 32) {
      double t = warp_tot[tid];
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const double v = __shfl_up_sync(0xffffffffu, t, s);
        if (tid >= s) t += v;
      }
      warp_tot[tid] = t;
    }
    __syncthreads();
    const double before = (tid >> 5) > 0 ? warp_tot[(tid >> 5) - 1] : 0.0;
    acc[i0] = before + (run - a1) + a0;
    acc[i0 + 1] = before + run;
  }
  if (tid == 0) { first_below = M; first_hit = M; first_draw = M; }
  __syncthreads();
  const double total = acc[M - 1];
  if (!(total > 0.0)) {
    if (tid == 0) out[blockIdx.x] = token_of(0);
    return;
  }
  int keep = M;
  if (o.min_p > 0.0) {
    const double th = o.min_p * ((double)probs[0] / total);
    for (int i = tid; i < M; i += SF_THREADS)
      if ((double)probs[i] / total < th) atomicMin(&first_below, i);
    __syncthreads();
    keep = first_below < 1 ? 1 : first_below;
  }
  const int top_k = (int)o.top_k;
  if (top_k > 0 && top_k < keep) keep = top_k;
  if (o.top_p < 1.0) {
    for (int i = tid; i < keep; i += SF_THREADS)
      if (acc[i] / total >= o.top_p) atomicMin(&first_hit, i);
    __syncthreads();
    if (first_hit < keep) keep = first_hit + 1;
  }
  const double r = o.u * acc[keep - 1];
  for (int i = tid; i < keep; i += SF_THREADS)
    if (acc[i] >= r) atomicMin(&first_draw, i);
  __syncthreads();
  if (tid == 0) out[blockIdx.x] = token_of(first_draw < keep ? first_draw : keep - 1);
}

// Penalties over a row's context (src/model.cpp:672-686).  counts[r] points to the row's token counts [V]
// (how often each token occurs in its context so far), or is null for a row without penalties.
__global__ void sample_penalties_kernel(float* __restrict__ logits, int V, const int* const* __restrict__ counts,
                                        const float* __restrict__ params /* [R, 3]: repetition, presence, frequency */) {
  const int row = blockIdx.y;
  const int* c = counts[row];
  if (c == nullptr) return;
  const int tok = blockIdx.x * blockDim.x + threadIdx.x;
  if (tok >= V) return;
  const int count = c[tok];
  if (count <= 0) return;
  const float rep = params[3 * row], presence = params[3 * row + 1], frequency = params[3 * row + 2];
  float x = logits[(int64_t)row * V + tok];
  if (rep != 1.0f) x = x > 0.0f ? __fdiv_rn(x, rep) : __fmul_rn(x, rep);
  if (presence != 0.0f) x = __fsub_rn(x, presence);
  if (frequency != 0.0f) x = __fsub_rn(x, __fmul_rn(frequency, (float)count));
  logits[(int64_t)row * V + tok] = x;
}

// The chosen tokens join their rows' contexts.
__global__ void sample_count_kernel(int* const* __restrict__ counts, const int* __restrict__ ids, int R, int V) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= R || counts[row] == nullptr) return;
  const int t = ids[row];
  if (t >= 0 && t < V) counts[row][t] += 1;
}

}  // namespace exl3

using namespace exl3;

// rows: float64 [R, 5] on the device: temperature (<= 0: greedy), top_k (0: off, at most 2048), top_p, min_p and
// the row's uniform number in [0, 1).  out: int32 [R].
extern "C" int exl3_sample_filtered(const float* logits, const double* rows, int* out, int R, int V,
                                    cudaStream_t stream) {
  if (R == 0) return 0;
  if (R < 0 || V < 1) { set_error("sample_filtered: bad sizes rows=%d vocab=%d", R, V); return ERR_BAD_ARGUMENT; }
  sample_filtered_kernel<<<R, SF_THREADS, 0, stream>>>(logits, reinterpret_cast<const SfRow*>(rows), out, V);
  return launch_status("sample_filtered");
}

extern "C" int exl3_sample_filtered_cap() { return SF_CAP; }

// counts: R device pointers (null: the row has no penalties) to int32 [V] token counts of the rows' contexts;
// params: float32 [R, 3] (repetition, presence, frequency penalty).  Changes logits in place.
extern "C" int exl3_sample_penalties(float* logits, int R, int V, const int* const* counts, const float* params,
                                     cudaStream_t stream) {
  if (R == 0) return 0;
  if (R < 0 || R > 65535 || V < 1) { set_error("sample_penalties: bad sizes rows=%d vocab=%d", R, V); return ERR_BAD_ARGUMENT; }
  sample_penalties_kernel<<<dim3(ceil_div(V, 256), R), 256, 0, stream>>>(logits, V, counts, params);
  return launch_status("sample_penalties");
}

// counts[r][ids[r]] += 1 for the rows that keep counts.
extern "C" int exl3_sample_count(int* const* counts, const int* ids, int R, int V, cudaStream_t stream) {
  if (R == 0) return 0;
  if (R < 0 || V < 1) { set_error("sample_count: bad sizes rows=%d vocab=%d", R, V); return ERR_BAD_ARGUMENT; }
  sample_count_kernel<<<ceil_div(R, 128), 128, 0, stream>>>(counts, ids, R, V);
  return launch_status("sample_count");
}
