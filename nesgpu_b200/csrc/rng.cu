// On-device noise set-up: Gaussian / uniform fills and per-member permutations (Philox-4x32-10).
#include "common.cuh"

namespace nes {

// Four normals from one Philox call (counter ctr): Box-Muller on two uniform pairs.  The hardware's approximate
// logarithm and sine / cosine are used: their absolute errors (~1e-6 on these ranges) are far below the
// resolution of the 24-bit uniforms that feed them, and the kernel is bound by its arithmetic, not by memory.
__device__ __forceinline__ void normal4(const Philox& ph, uint64_t ctr, float mean, float std, float (&z)[4]) {
  uint32_t r[4];
  ph.rounds<7>(uint32_t(ctr), uint32_t(ctr >> 32), 0u, 0u, r);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float u1 = u32_to_unit(r[2 * h]);
    const float u2 = u32_to_unit(r[2 * h + 1]);
    const float rad = sqrtf(-2.0f * __logf(u1));
    float s, c;
    __sincosf(fmaf(6.283185307179586f, u2, -3.141592653589793f), &s, &c);      // angle in (-pi, pi]: the accurate range
    z[2 * h] = fmaf(std, rad * c, mean);
    z[2 * h + 1] = fmaf(std, rad * s, mean);
  }
}

// A thread owns two groups of four outputs, one block-width apart (two independent Philox chains in flight, two
// coalesced 128-bit stores).  Group g always uses counter offset + g, whatever the launch shape.
template <bool VEC>
__global__ void __launch_bounds__(256) fill_normal_kernel(float* __restrict__ out, int64_t n, float mean, float std,
                                                          uint64_t seed, uint64_t offset) {
  const int64_t g0 = (int64_t(blockIdx.x) * 2) * blockDim.x + threadIdx.x;
  const int64_t g1 = g0 + blockDim.x;
  const Philox ph(seed);
  float za[4], zb[4];
  if (g0 * 4 >= n) return;
  normal4(ph, offset + uint64_t(g0), mean, std, za);
  const bool second = g1 * 4 < n;
  if (second) normal4(ph, offset + uint64_t(g1), mean, std, zb);
  if (VEC && g0 * 4 + 3 < n) {
    __stcs(reinterpret_cast<float4*>(out) + g0, make_float4(za[0], za[1], za[2], za[3]));
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) if (g0 * 4 + j < n) out[g0 * 4 + j] = za[j];
  }
  if (!second) return;
  if (VEC && g1 * 4 + 3 < n) {
    __stcs(reinterpret_cast<float4*>(out) + g1, make_float4(zb[0], zb[1], zb[2], zb[3]));
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) if (g1 * 4 + j < n) out[g1 * 4 + j] = zb[j];
  }
}

__global__ void fill_uniform_kernel(float* __restrict__ out, int64_t n, float lo, float hi,
                                    uint64_t seed, uint64_t offset) {
  const int64_t q = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (q * 4 >= n) return;
  const uint64_t ctr = offset + uint64_t(q);
  uint32_t r[4];
  Philox ph(seed);
  ph(uint32_t(ctr), uint32_t(ctr >> 32), 0u, 2u, r);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (q * 4 + j < n) out[q * 4 + j] = fmaf(hi - lo, u32_to_unit(r[j]), lo);
}

// One block per member: draw a 32-bit key per position, sort (key, position) pairs with a
// bitonic network in shared memory, emit the positions of the `keep` smallest keys.  Ties in
// the key are broken by position (probability ~ n^2 / 2^33 per member).
__global__ void sample_permutations_kernel(int16_t* __restrict__ out, int n, int n_pow2, int keep, uint64_t seed,
                                           int64_t first_member) {
  extern __shared__ __align__(16) unsigned char dyn[];
  uint64_t* keys = reinterpret_cast<uint64_t*>(dyn);
  const int64_t d = blockIdx.x;
  const uint64_t member = uint64_t(first_member + d);      // the draw depends on the global member index only
  Philox ph(seed);
  for (int q = threadIdx.x; q * 4 < n_pow2; q += blockDim.x) {
    uint32_t r[4];
    ph(uint32_t(q), uint32_t(member), uint32_t(member >> 32), 1u, r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = q * 4 + j;
      if (i < n_pow2) keys[i] = (i < n) ? ((uint64_t(r[j]) << 16) | uint64_t(i)) : ~uint64_t(0);
    }
  }
  __syncthreads();
  for (int size = 2; size <= n_pow2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < n_pow2 / 2; i += blockDim.x) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool up = ((lo & size) == 0);
        const uint64_t a = keys[lo], b = keys[hi];
        if ((a > b) == up) { keys[lo] = b; keys[hi] = a; }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < keep; i += blockDim.x) out[d * keep + i] = int16_t(keys[i] & 0xFFFFu);
}

__global__ void sample_indices_kernel(int16_t* __restrict__ out, int64_t total, int n, uint64_t seed, uint64_t offset) {
  const int64_t q = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (q * 4 >= total) return;
  uint32_t r[4];
  Philox ph(seed);
  const uint64_t ctr = offset + uint64_t(q);
  ph(uint32_t(ctr), uint32_t(ctr >> 32), 0u, 3u, r);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (q * 4 + j < total) out[q * 4 + j] = int16_t((uint64_t(r[j]) * uint64_t(n)) >> 32);
}

__global__ void fill_signs_kernel(int8_t* __restrict__ out, int64_t n, uint64_t seed, uint64_t offset) {
  const int64_t q = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;    // 128 outputs per thread
  if (q * 128 >= n) return;
  const uint64_t ctr = offset + uint64_t(q);
  uint32_t r[4];
  Philox ph(seed);
  ph(uint32_t(ctr), uint32_t(ctr >> 32), 0u, 4u, r);
  for (int j = 0; j < 128; ++j)
    if (q * 128 + j < n) out[q * 128 + j] = ((r[j >> 5] >> (j & 31)) & 1u) ? int8_t(1) : int8_t(-1);
}

}  // namespace nes

using namespace nes;

extern "C" int nes_fill_signs(int8_t* out, int64_t n, uint64_t seed, uint64_t offset, nes_stream_t stream) {
  NES_REQUIRE(n >= 0, NES_ERR_BAD_ARG, "fill_signs: negative extent");
  if (n == 0) return NES_OK;
  NES_REQUIRE(out, NES_ERR_BAD_ARG, "fill_signs: null pointer");
  const int64_t groups = ceil_div<int64_t>(n, 128);
  fill_signs_kernel<<<(unsigned)ceil_div<int64_t>(groups, 128), 128, 0, as_stream(stream)>>>(out, n, seed, offset);
  return check_launch("fill_signs");
}

extern "C" int nes_fill_normal(float* out, int64_t n, float mean, float std, uint64_t seed, uint64_t offset,
                               nes_stream_t stream) {
  NES_REQUIRE(n >= 0, NES_ERR_BAD_ARG, "fill_normal: negative extent");
  if (n == 0) return NES_OK;
  NES_REQUIRE(out, NES_ERR_BAD_ARG, "fill_normal: null pointer");
  const int64_t groups = ceil_div<int64_t>(n, 4);
  NES_REQUIRE(ceil_div<int64_t>(groups, 512) <= INT32_MAX, NES_ERR_UNSUPPORTED, "fill_normal: n too large");
  const unsigned blocks = (unsigned)ceil_div<int64_t>(groups, 512);
  if (aligned16(out)) fill_normal_kernel<true><<<blocks, 256, 0, as_stream(stream)>>>(out, n, mean, std, seed, offset);
  else fill_normal_kernel<false><<<blocks, 256, 0, as_stream(stream)>>>(out, n, mean, std, seed, offset);
  return check_launch("fill_normal");
}

extern "C" int nes_fill_uniform(float* out, int64_t n, float lo, float hi, uint64_t seed, uint64_t offset,
                                nes_stream_t stream) {
  NES_REQUIRE(n >= 0, NES_ERR_BAD_ARG, "fill_uniform: negative extent");
  if (n == 0) return NES_OK;
  NES_REQUIRE(out, NES_ERR_BAD_ARG, "fill_uniform: null pointer");
  const int64_t groups = ceil_div<int64_t>(n, 4);
  NES_REQUIRE(ceil_div<int64_t>(groups, 256) <= INT32_MAX, NES_ERR_UNSUPPORTED, "fill_uniform: n too large");
  fill_uniform_kernel<<<(unsigned)ceil_div<int64_t>(groups, 256), 256, 0, as_stream(stream)>>>(out, n, lo, hi, seed, offset);
  return check_launch("fill_uniform");
}

extern "C" int nes_sample_permutations(int16_t* out, int64_t D, int n, int keep, int with_replacement,
                                       uint64_t seed, int64_t first_member, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && n > 0 && keep >= 0 && first_member >= 0, NES_ERR_BAD_ARG, "sample_permutations: bad extent");
  NES_REQUIRE(n <= 32767, NES_ERR_UNSUPPORTED, "sample_permutations: n=%d does not fit int16", n);
  if (D == 0 || keep == 0) return NES_OK;
  NES_REQUIRE(out, NES_ERR_BAD_ARG, "sample_permutations: null pointer");
  cudaStream_t st = as_stream(stream);
  if (with_replacement) {
    const int64_t total = D * keep;
    sample_indices_kernel<<<(unsigned)ceil_div<int64_t>(ceil_div<int64_t>(total, 4), 256), 256, 0, st>>>(out, total, n, seed,
                                                                                                      uint64_t(first_member) * uint64_t(ceil_div(keep, 4) + 1));
    return check_launch("sample_permutations(indices)");
  }
  NES_REQUIRE(keep <= n, NES_ERR_BAD_ARG, "sample_permutations: keep > n without replacement");
  NES_REQUIRE(n <= 16384, NES_ERR_UNSUPPORTED, "sample_permutations: n=%d > 16384 not implemented", n);
  NES_REQUIRE(D <= INT32_MAX, NES_ERR_UNSUPPORTED, "sample_permutations: D too large");
  int n_pow2 = 1;
  while (n_pow2 < n) n_pow2 <<= 1;
  const size_t smem = size_t(n_pow2) * sizeof(uint64_t);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(sample_permutations_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(NES_ERR_UNSUPPORTED, "sample_permutations: %zu B of shared memory refused", smem);
  }
  const int threads = n_pow2 / 2 < 32 ? 32 : (n_pow2 / 2 > 512 ? 512 : n_pow2 / 2);
  sample_permutations_kernel<<<(unsigned)D, threads, smem, st>>>(out, n, n_pow2, keep, seed, first_member);
  return check_launch("sample_permutations");
}
