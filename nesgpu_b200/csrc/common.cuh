// Shared helpers for the sm_100a kernels behind include/nesgpu_b200.h.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/nesgpu_b200.h"

namespace nes {

// Thread-local text of the last failure; returned by nes_last_error().
char* last_error_buffer();
int fail(int status, const char* fmt, ...);

inline cudaStream_t as_stream(nes_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Number of kernel launches this library has issued in the process (diagnostic).
void count_launch();

inline int check_launch(const char* what) {
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return NES_OK;
}

template <typename T>
__host__ __device__ constexpr T ceil_div(T a, T b) { return (a + b - 1) / b; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (148 on B200), cached per device.
int sm_count();

#define NES_REQUIRE(cond, status, ...) \
  do { if (!(cond)) return ::nes::fail(status, __VA_ARGS__); } while (0)

// ---------------------------------------------------------------- Philox-4x32-10
struct Philox {
  uint32_t k0, k1;
  __host__ __device__ Philox(uint64_t seed) : k0(uint32_t(seed)), k1(uint32_t(seed >> 32)) {}
  __host__ __device__ static inline void mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
#ifdef __CUDA_ARCH__
    lo = a * b; hi = __umulhi(a, b);
#else
    uint64_t p = uint64_t(a) * b; lo = uint32_t(p); hi = uint32_t(p >> 32);
#endif
  }
  // counter = (c0..c3); returns four 32-bit words in r[0..3]
  __host__ __device__ inline void operator()(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                             uint32_t r[4]) const {
    rounds<10>(c0, c1, c2, c3, r);
  }
  // The same generator with ROUNDS rounds.  Ten is the customary conservative choice; seven is the smallest
  // count its authors report as passing the BigCrush battery, and is what the bulk Gaussian fill uses
  // (that kernel is bound by its integer arithmetic).
  template <int ROUNDS>
  __host__ __device__ inline void rounds(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t r[4]) const {
    uint32_t a = k0, b = k1;
#pragma unroll
    for (int i = 0; i < ROUNDS; ++i) {
      uint32_t hi0, lo0, hi1, lo1;
      mulhilo(0xD2511F53u, c0, hi0, lo0);
      mulhilo(0xCD9E8D57u, c2, hi1, lo1);
      uint32_t n0 = hi1 ^ c1 ^ a, n1 = lo1, n2 = hi0 ^ c3 ^ b, n3 = lo0;
      c0 = n0; c1 = n1; c2 = n2; c3 = n3;
      a += 0x9E3779B9u; b += 0xBB67AE85u;
    }
    r[0] = c0; r[1] = c1; r[2] = c2; r[3] = c3;
  }
};

// 32 random bits -> uniform in (0, 1]
__host__ __device__ inline float u32_to_unit(uint32_t x) {
  return (float(x >> 8) + 1.0f) * (1.0f / 16777216.0f);
}

// antithetic sign of repeat r (modules/base.py:377-378): -1 for r >= (R+1)/2
__host__ __device__ inline float anti_sign(int64_t r, int64_t R, int antithetic) {
  return (antithetic && r >= (R + 1) / 2) ? -1.0f : 1.0f;
}

}  // namespace nes
