// An argmax entry point that allocates nothing.  It has no counterpart in the
// reference (which picks tokens on the host, src/model.cpp:688-696); it exists
// for callers of this library that are not allowed to allocate device memory.
//
// Who that is: a host program that has handed all of the GPU's memory to its
// own pool at start-up, so that a later cudaMalloc simply fails; a thread on a
// latency budget that must not enter the driver's allocator, which may take a
// device-wide lock or wait for the device; plug-in style code that gets
// buffers from its host application and is forbidden to create its own.  The
// ordinary entry point, exl3_argmax, needs the caller to bring scratch memory
// for vocabularies above 4096; this one brings its own.
//
// The scratch is a fixed array in device memory that is part of the library
// image: every GPU that loads the library holds EXL3_ARGMAX_STATIC_BYTES
// (128 KiB) of it until the process exits.  Limits that follow from its size:
// rows <= EXL3_ARGMAX_STATIC_MAX_ROWS and vocab <= EXL3_ARGMAX_STATIC_MAX_VOCAB;
// larger requests are refused with an error, never truncated.
//
// The first call on each device looks up the array's device address (with that
// device current) and remembers it; make that first call before you begin any
// stream capture on the device.  Later calls only launch kernels.
//
// All calls share the one array and it keeps what the last call left.  Nothing
// in it has to start at zero: each call overwrites every entry it later reads.
// Two calls that can run on the GPU at the same time (different streams, or
// different threads without ordering) race on it and give wrong tokens; order
// them on one stream or with events.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#define EXL3_ARGMAX_STATIC_MAX_ROWS 64
#define EXL3_ARGMAX_STATIC_MAX_VOCAB 524288
#define EXL3_ARGMAX_STATIC_BYTES (64 * 256 * 8)

extern "C" {
// out[r] = index of the first maximum of logits[r, 0..V-1]; float32 logits
// [R, V] and int32 out [R] are the caller's device buffers.  Returns 0, a
// cudaError_t (> 0) or a negative code as the other entry points do;
// exl3_last_error() has the message.
int exl3_argmax_static(const float* logits, int* out, int R, int V, cudaStream_t stream);
}
