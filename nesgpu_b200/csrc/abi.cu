// Status reporting and device queries shared by all entry points.
#include <stdarg.h>
#include <string.h>
#include "common.cuh"

namespace nes {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return status;
}

static unsigned long long g_launches = 0;
void count_launch() { __atomic_fetch_add(&g_launches, 1ULL, __ATOMIC_RELAXED); }
unsigned long long launches() { return __atomic_load_n(&g_launches, __ATOMIC_RELAXED); }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace nes

extern "C" int nes_abi_version(void) { return NES_ABI_VERSION; }

extern "C" const char* nes_status_string(int status) {
  switch (status) {
    case NES_OK: return "ok";
    case NES_ERR_BAD_ARG: return "bad argument";
    case NES_ERR_UNSUPPORTED: return "unsupported size or option";
    case NES_ERR_LAUNCH: return "CUDA launch error";
    case NES_ERR_TIMEOUT: return "device-side wait timed out";
    case NES_ERR_SCRATCH: return "scratch buffer missing or too small";
    default: return "unknown status";
  }
}

extern "C" const char* nes_last_error(void) { return nes::last_error_buffer(); }

extern "C" int64_t nes_launch_count(void) { return (int64_t)nes::launches(); }
