// Picking the next token on the device.
//
// argmax: the first maximum wins, as in the reference's strict ">" scans
// (src/model.cpp:604-613, 688-696).  Sampling with temperature and filters
// is in sampling_filtered.cu.
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace exl3 {

constexpr int SAMPLE_THREADS = 1024;

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const float* row = logits + (int64_t)blockIdx.x * V;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (bi == 0x7fffffff && !(v != v))) { best = v; bi = i; }   // ascending i: first max kept
  }
  auto better = [](float v, int i, float bv, int b) { return v > bv || (v == bv && i < b); };
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = sv[lane];
    bi = si[lane];
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
  }
}

// Two stages for large vocabularies: blocks of ARGMAX_CHUNK logits each leave
// their first maximum in scratch, then one block per row picks among those.
constexpr int ARGMAX_CHUNK = 2048;
constexpr int ARGMAX_THREADS = 256;

__device__ inline bool argmax_better(float v, int i, float bv, int b) { return v > bv || (v == bv && i < b); }

__device__ inline void argmax_block_reduce(float& best, int& bi, float* sv, int* si) {
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (argmax_better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = lane < nwarps ? sv[lane] : -INFINITY;
    bi = lane < nwarps ? si[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (argmax_better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
  }
}

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_partial_kernel(const float* __restrict__ logits, float* __restrict__ pv, int* __restrict__ pi, int V,
                      int nchunks) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.y, chunk = blockIdx.x;
  const float* p = logits + (int64_t)row * V;
  const int b = chunk * ARGMAX_CHUNK, e = min(V, b + ARGMAX_CHUNK);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = b + threadIdx.x; i < e; i += blockDim.x) {
    const float v = __ldcg(p + i);
    if (v > best || (bi == 0x7fffffff && !(v != v))) { best = v; bi = i; }
  }
  argmax_block_reduce(best, bi, sv, si);
  if (threadIdx.x == 0) { pv[(int64_t)row * nchunks + chunk] = best; pi[(int64_t)row * nchunks + chunk] = bi; }
}

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int* __restrict__ out, int nchunks) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {
    const float v = __ldcg(pv + (int64_t)row * nchunks + c);
    const int i = __ldcg(pi + (int64_t)row * nchunks + c);
    if (i != 0x7fffffff && (bi == 0x7fffffff || argmax_better(v, i, best, bi))) { best = v; bi = i; }
  }
  argmax_block_reduce(best, bi, sv, si);
  if (threadIdx.x == 0) out[row] = (bi == 0x7fffffff) ? 0 : bi;
}

}  // namespace exl3

using namespace exl3;

extern "C" size_t exl3_argmax_scratch_bytes(int R, int V) {
  if (V <= 2 * ARGMAX_CHUNK) return 0;
  return (size_t)R * ceil_div(V, ARGMAX_CHUNK) * (sizeof(float) + sizeof(int));
}

// scratch may be null: then, and for small vocabularies, one block per row scans the whole row.
extern "C" int exl3_argmax(const float* logits, int* out, int R, int V, void* scratch, size_t scratch_bytes,
                           cudaStream_t stream) {
  if (R == 0) return 0;
  if (R < 0 || V < 1) { set_error("argmax: bad sizes rows=%d vocab=%d", R, V); return ERR_BAD_ARGUMENT; }
  const size_t need = exl3_argmax_scratch_bytes(R, V);
  if (need == 0 || scratch == nullptr) {
    argmax_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, out, V);
    return launch_status("argmax");
  }
  if (scratch_bytes < need) {
    set_error("argmax: scratch of %zu bytes is too small, need %zu", scratch_bytes, need);
    return ERR_SCRATCH;
  }
  if (R > 65535) { set_error("argmax: too many rows (%d)", R); return ERR_UNSUPPORTED; }
  const int nchunks = ceil_div(V, ARGMAX_CHUNK);
  float* pv = static_cast<float*>(scratch);
  int* pi = reinterpret_cast<int*>(pv + (size_t)R * nchunks);
  launch_pdl(argmax_partial_kernel, dim3(nchunks, R), dim3(ARGMAX_THREADS), 0, stream, logits, pv, pi, V, nchunks);
  int rc = launch_status("argmax_partial");
  if (rc) return rc;
  launch_pdl(argmax_final_kernel, dim3(R), dim3(ARGMAX_THREADS), 0, stream, (const float*)pv, (const int*)pi, out,
             nchunks);
  return launch_status("argmax_final");
}

// ---------------------------------------------------------------------------
// The entry point that allocates nothing (see no_alloc.h).
// ---------------------------------------------------------------------------
#include "no_alloc.h"

#include <mutex>

namespace exl3 {

// Partial maxima for up to 64 rows x 256 chunks of 2048 logits: 64 * 256 floats,
// then 64 * 256 ints.  In host code this name is only a handle for
// cudaGetSymbolAddress, not a device address.
static __device__ __align__(256) unsigned char g_argmax_static_scratch[EXL3_ARGMAX_STATIC_BYTES];

constexpr int STATIC_MAX_DEVICES = 64;
static void* g_static_scratch_ptr[STATIC_MAX_DEVICES] = {};
static std::mutex g_static_scratch_mutex;

// The device address of the array on the current device, looked up once per device.
static int static_scratch(void** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_error("argmax_static: cudaGetDevice failed: %s", cudaGetErrorString(e)); return (int)e; }
  if (dev < 0 || dev >= STATIC_MAX_DEVICES) { set_error("argmax_static: device %d is out of range", dev); return ERR_UNSUPPORTED; }
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_argmax_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("argmax_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : ERR_UNSUPPORTED;
    }
    g_static_scratch_ptr[dev] = p;
  }
  *ptr = g_static_scratch_ptr[dev];
  return 0;
}

}  // namespace exl3

extern "C" int exl3_argmax_static(const float* logits, int* out, int R, int V, cudaStream_t stream) {
  if (R == 0) return 0;
  if (R < 0 || V < 1) { set_error("argmax_static: bad sizes rows=%d vocab=%d", R, V); return ERR_BAD_ARGUMENT; }
  if (R > EXL3_ARGMAX_STATIC_MAX_ROWS || V > EXL3_ARGMAX_STATIC_MAX_VOCAB) {
    set_error("argmax_static: rows=%d vocab=%d exceed the built-in scratch (at most %d rows, vocab %d)", R, V,
              EXL3_ARGMAX_STATIC_MAX_ROWS, EXL3_ARGMAX_STATIC_MAX_VOCAB);
    return ERR_SCRATCH;
  }
  void* scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc) return rc;
  // Same two kernels as exl3_argmax, for every vocabulary size, so that the
  // array is what the second kernel reads.  Every (row, chunk) entry that the
  // second kernel reads is written by the first in this call.
  const int nchunks = ceil_div(V, ARGMAX_CHUNK);
  float* pv = static_cast<float*>(scratch);
  int* pi = reinterpret_cast<int*>(pv + (size_t)R * nchunks);
  launch_pdl(argmax_partial_kernel, dim3(nchunks, R), dim3(ARGMAX_THREADS), 0, stream, logits, pv, pi, V, nchunks);
  rc = launch_status("argmax_static (partial)");
  if (rc) return rc;
  launch_pdl(argmax_final_kernel, dim3(R), dim3(ARGMAX_THREADS), 0, stream, (const float*)pv, (const int*)pi, out,
             nchunks);
  return launch_status("argmax_static (final)");
}
