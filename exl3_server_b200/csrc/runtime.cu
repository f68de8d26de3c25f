// Error channel shared by the entry points.
#include "api.h"
#include "common.cuh"

#include <atomic>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

namespace exl3 {

static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("EXL3_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

}  // namespace exl3

extern "C" const char* exl3_last_error() { return exl3::g_error; }
extern "C" int exl3_abi_version() { return 5; }
// Kernel launches made through this library since it was loaded (launches
// recorded into a CUDA graph count once, when they are captured).
extern "C" long long exl3_launch_count() { return exl3::g_launches.load(std::memory_order_relaxed); }
