// Shared device helpers for the sm_100a kernels: element types, 16-byte vector
// access, warp and block reductions with a fixed order, and the error channel
// of the C entry points.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace exl3 {

// Element type codes used by every C entry point.
enum : int { DT_F32 = 0, DT_BF16 = 1 };

// Error channel: entry points return 0, a cudaError_t (> 0) or one of these (< 0).
enum : int {
  ERR_BAD_ARGUMENT = -1,   // a size or flag this kernel does not accept
  ERR_UNSUPPORTED = -2,    // a valid size that no kernel variant covers
  ERR_ALIGNMENT = -3,      // a pointer or stride that breaks a vector-access rule
  ERR_SCRATCH = -4,        // scratch memory too small for the request
};

void set_error(const char* fmt, ...);

template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int code = DT_F32;
  static constexpr int vec = 4;            // elements in 16 bytes
  __device__ static inline float load(const float* p) { return *p; }
  __device__ static inline void store(float* p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int code = DT_BF16;
  static constexpr int vec = 8;
  __device__ static inline float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static inline void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// 16 bytes of T widened to floats (p must be 16-byte aligned).
__device__ inline void load_vec(const float* p, float (&v)[4]) {
  float4 r = *reinterpret_cast<const float4*>(p);
  v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}
__device__ inline void load_vec(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 r = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
// The same through L2 only.  Kernels launched with programmatic dependent
// launch overlap their predecessors on an SM, so L1 may still hold a line of a
// buffer from before its producer rewrote it; everything a step's kernels
// hand to each other is read this way.  Weights may use any load.
__device__ inline void load_vec_cg(const float* p, float (&v)[4]) {
  float4 r = __ldcg(reinterpret_cast<const float4*>(p));
  v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}
__device__ inline void load_vec_cg(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 r = __ldcg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
// 16 raw bytes through L2 only, and their widening to floats afterwards: lets a
// kernel put several loads in flight before it uses the first.
__device__ inline uint4 load_raw_cg(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ inline void unpack_raw(const uint4& r, float (&v)[4], const float*) {
  v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
}
__device__ inline void unpack_raw(const uint4& r, float (&v)[8], const __nv_bfloat16*) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ inline void store_vec(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ inline void store_vec(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 r;
  uint32_t* w = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = r;
}

__device__ inline float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order depends only on blockDim, never on the data or the grid.
__device__ inline float block_sum(float v, float* smem32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? smem32[lane] : 0.0f;
  t = warp_sum(t);
  return t;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Called after every launch by the entry points.
int launch_status(const char* what);

// Programmatic dependent launch.  A kernel launched with launch_pdl may start
// while the kernel before it in the stream is still running; it must call
// pdl_wait() before it reads anything that kernel wrote and before it writes
// anything at all.  What comes before pdl_wait() may only touch data that no
// kernel of the step writes (weights).  pdl_trigger() lets the next kernel in
// the stream start early in the same way.  Without the launch attribute both
// calls do nothing.
__device__ inline void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ inline void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();

// Sine and cosine of the rotary angle p * f of position p, where the frequency f is given as a float32 (hi) and,
// optionally, what float32 lost of it (lo; 0 without).  The product's own rounding error comes back through one
// fma, so the angle is right to a few 1e-9 of itself, not to 6e-8: at position 1,000 that is the difference between
// 1e-6 and 5e-5 radians in the fastest pairs, and it grows with the position.
__device__ inline void rope_sincos(float p, float hi, float lo, float* sn, float* cs) {
  const float a = p * hi;
  const float d = fmaf(p, hi, -a) + p * lo;              // what a misses of the angle: below 0.02 up to position 300,000
  float s, c;
  sincosf(a, &s, &c);
  const float d2 = d * d;
  const float sd = d * fmaf(d2, -1.0f / 6.0f, 1.0f), cd = fmaf(d2, -0.5f, 1.0f);   // sin d and cos d, good to 1e-8 there
  *sn = fmaf(s, cd, c * sd);
  *cs = fmaf(c, cd, -s * sd);
}

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);     // errors are read by launch_status()
}

// The same with the grid's blocks in thread-block clusters of `cluster` along x.
template <typename... KArgs, typename... Args>
inline void launch_pdl_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster, size_t smem,
                                cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);     // errors are read by launch_status()
}

}  // namespace exl3
