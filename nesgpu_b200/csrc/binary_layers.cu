// Layer-level entry points of the bit-packed population layers (modules/binary.py of the reference):
// everything a BinarizedLinear / BinarizedConv2d does around the XOR-popcount product -- Bernoulli
// probabilities, bias noise, centring of the fitness, l1 / l2 terms, the bias gradient, the
// `2 * counts - n` activation, the fp16 thresholds (with or without the batch mean) and the packing of
// the resulting bits for the next layer -- as kernels, so that the Python layer classes only launch.
//
// Half-precision steps follow the reference's tensor arithmetic operation by operation: each of its fp16
// tensor ops rounds once to fp16 (computed in fp32), sums over fp16 values accumulate in fp32.  Where the
// activations are integers below 2^24 in magnitude the fp32 sums are exact, so the batch-mean thresholds
// do not depend on the order of summation and the thresholded bits are reproducible bit for bit.
#include "common.cuh"

namespace nes {

int bin_weighted_sum_impl(const void* in, const uint16_t* w_half, uint16_t* out_half, int64_t D, int64_t rows,
                          int64_t words, int64_t zbits, int word_bits, void* scratch, int64_t scratch_bytes,
                          cudaStream_t st);

// ---- N = 1 product (one packed input vector per member) with the layer's epilogues ---------------------
//
// HBM-bound: the member's weight rows are streamed once.  Four or eight lanes share a row (at 1024-bit rows:
// eight lanes, one 16-byte chunk each, so a warp-wide load reads four whole rows = 512 contiguous bytes), a
// warp covers a group of 32 rows in as many passes as lanes share a row, with all loads issued before the
// first use; the member's input chunks sit in registers, and after a butterfly over the sharing lanes the
// counts are dealt back so that lane L owns row L of the group: stores are coalesced and one __ballot_sync
// yields 32 packed output bits.
enum { BMV_COUNTS = 0, BMV_ACT = 1, BMV_BOOL = 2, BMV_PACKED = 3 };

// One group = 32 consecutive rows of one member, handled by one warp.  LPR lanes share a row (lane % LPR takes
// chunks sub, sub + LPR, ...), so a warp-wide load covers 32 / LPR rows: with LPR * 16 bytes = the row length
// every load instruction reads one contiguous span of whole rows.
template <int LPR, int CPL>
struct BmvGroup {
  static constexpr int RPP = 32 / LPR;          // rows per pass
  uint4 xv[CPL];
  uint4 av[LPR][CPL];
  int64_t z, base;

  __device__ __forceinline__ void load(const uint4* __restrict__ A, const uint4* __restrict__ X, int64_t g, int64_t gpm, int64_t M,
                                       int cpr, int lane) {
    const int sub = lane % LPR, rl = lane / LPR;
    z = g / gpm;
    base = (g - z * gpm) * 32;
#pragma unroll
    for (int j = 0; j < CPL; ++j) {
      const int c = sub + LPR * j;
      xv[j] = (c < cpr) ? __ldg(X + z * cpr + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < LPR; ++i) {
      const int64_t m = base + RPP * i + rl;
      const uint4* row = A + (z * M + m) * cpr;
#pragma unroll
      for (int j = 0; j < CPL; ++j) {
        const int c = sub + LPR * j;
        av[i][j] = (m < M && c < cpr) ? __ldcs(row + c) : xv[j];      // padding contributes popc(x ^ x) = 0
      }
    }
  }

  // the count of row base + lane, in every lane
  __device__ __forceinline__ int reduce(int lane) const {
    int mine = 0;
#pragma unroll
    for (int i = 0; i < LPR; ++i) {
      int s = 0;
#pragma unroll
      for (int j = 0; j < CPL; ++j)
        s += __popc(av[i][j].x ^ xv[j].x) + __popc(av[i][j].y ^ xv[j].y) + __popc(av[i][j].z ^ xv[j].z) + __popc(av[i][j].w ^ xv[j].w);
#pragma unroll
      for (int sh = 1; sh < LPR; sh <<= 1) s += __shfl_xor_sync(0xffffffffu, s, sh);
      const int v = __shfl_sync(0xffffffffu, s, LPR * (lane % RPP));   // row RPP * i + (lane % RPP) of this pass
      if (lane / RPP == i) mine = v;
    }
    return mine;
  }
};

template <int MODE>
__device__ __forceinline__ void bmv_store(void* __restrict__ out, const __half* __restrict__ bias, const __half* __restrict__ bias_noise,
                                          int64_t z, int64_t base, int lane, int64_t M, int count, int n_bits, int64_t out_row_u32) {
  const int64_t m = base + lane;
  const bool ok = m < M;
  if (MODE == BMV_COUNTS) {
    if (ok) static_cast<int32_t*>(out)[z * M + m] = count;
  } else if (MODE == BMV_ACT) {
    if (ok) static_cast<int32_t*>(out)[z * M + m] = 2 * count - n_bits;
  } else {
    bool bit = false;
    if (ok) {
      const __half th = __hadd(bias[m], bias_noise[z * M + m]);
      bit = __hgt(__int2half_rn(2 * count - n_bits), th);
    }
    if (MODE == BMV_BOOL) {
      if (ok) static_cast<uint8_t*>(out)[z * M + m] = uint8_t(bit);
    } else {
      const uint32_t word = __ballot_sync(0xffffffffu, bit);
      if (lane == 0) static_cast<uint32_t*>(out)[z * out_row_u32 + base / 32] = word;
    }
  }
}

// The grid is a few blocks per SM; every warp walks groups g = warp, warp + W, ... two at a time, so that the loads
// of two groups (sixteen 16-byte loads per lane at 1024-bit rows) are in flight before the first popcount.
template <int MODE, int LPR, int CPL>
__global__ void __launch_bounds__(256) bmv_rows_kernel(const uint4* __restrict__ A, const uint4* __restrict__ X,
                                                       void* __restrict__ out, const __half* __restrict__ bias,
                                                       const __half* __restrict__ bias_noise, int64_t M, int cpr,
                                                       int n_bits, int64_t out_row_u32, int64_t gpm, int64_t groups) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t W = int64_t(gridDim.x) * 8;
  for (int64_t g = int64_t(blockIdx.x) * 8 + warp; g < groups; g += 2 * W) {
    BmvGroup<LPR, CPL> a, b;
    a.load(A, X, g, gpm, M, cpr, lane);
    const bool two = g + W < groups;                    // uniform over the warp
    if (two) b.load(A, X, g + W, gpm, M, cpr, lane);
    bmv_store<MODE>(out, bias, bias_noise, a.z, a.base, lane, M, a.reduce(lane), n_bits, out_row_u32);
    if (two) bmv_store<MODE>(out, bias, bias_noise, b.z, b.base, lane, M, b.reduce(lane), n_bits, out_row_u32);
  }
}

// ---- column sums of the fp16-rounded activation ---------------------------------------------------------
// act (P, S, N) int32 (or counts with act = 2*c - offset).  sums[(shared ? 0 : p), n] = sum over s (and over p
// when shared) of float(half(act)).  One block per (32 columns, p or the whole batch).
__global__ void __launch_bounds__(256) act_colsum_kernel(const int32_t* __restrict__ act, float* __restrict__ sums,
                                                         int64_t P, int64_t S, int64_t N, int is_counts, int offset, int shared) {
  __shared__ float red[256];
  const int t = threadIdx.x, lane = t & 31, grp = t >> 5;
  const int64_t n = int64_t(blockIdx.x) * 32 + lane;
  const int64_t p0 = shared ? 0 : blockIdx.y, p1 = shared ? P : p0 + 1;
  float acc = 0.f;
  if (n < N) {
    const int64_t rows = (p1 - p0) * S;
    const int32_t* src = act + p0 * S * N + n;
#pragma unroll 4
    for (int64_t r = grp; r < rows; r += 8) {
      int a = src[r * N];
      if (is_counts) a = 2 * a - offset;
      acc += __half2float(__int2half_rn(a));
    }
  }
  red[t] = acc;
  __syncthreads();
  if (t < 32 && n < N) {
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) s += red[u * 32 + t];
    sums[(shared ? 0 : int64_t(blockIdx.y)) * N + n] = s;
  }
}

// ---- threshold: bit = half(act) > half(bias + bias_noise [+ half(mean)]) -----------------------------
// act (P, S, N); bias (N) fp16; bias_noise (P, N) fp16; sums as produced above (count = number of summed
// values).  Output: bool bytes (P, S, N), or bits packed along N into 32-bit units, row length out_row_u32
// (little-endian, so the same bytes serve int32 and int64 words).
template <bool PACKED>
__global__ void __launch_bounds__(256) act_threshold_kernel(const int32_t* __restrict__ act, const __half* __restrict__ bias,
                                                            const __half* __restrict__ bias_noise, const float* __restrict__ sums,
                                                            void* __restrict__ out, int64_t P, int64_t S, int64_t N,
                                                            int is_counts, int offset, int shared, float count,
                                                            int64_t out_row_u32) {
  const int lane = threadIdx.x & 31;
  const int64_t n32 = (N + 31) / 32;                         // 32-column groups per (p, s) row
  const int64_t g = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;       // one warp per group
  if (g >= P * S * n32) return;
  const int64_t row = g / n32, n = (g - row * n32) * 32 + lane;
  const int64_t p = row / S;
  bool bit = false;
  if (n < N) {
    int a = act[row * N + n];
    if (is_counts) a = 2 * a - offset;
    __half th = __hadd(bias[n], bias_noise[p * N + n]);
    if (sums) th = __hadd(th, __float2half_rn(sums[(shared ? 0 : p) * N + n] / count));
    bit = __hgt(__int2half_rn(a), th);
  }
  if (PACKED) {
    const uint32_t word = __ballot_sync(0xffffffffu, bit);
    if (lane == 0) static_cast<uint32_t*>(out)[row * out_row_u32 + (g - row * n32)] = word;
  } else if (n < N) {
    static_cast<uint8_t*>(out)[row * N + n] = uint8_t(bit);
  }
}

// act = 2 * counts - offset (may run in place)
__global__ void act_from_counts_kernel(const int32_t* __restrict__ counts, int32_t* __restrict__ act, int64_t n, int offset) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e < n) act[e] = 2 * counts[e] - offset;
}

// trunc(half(bias + bias_noise)) + offset as int32: the integer threshold of the reference's conv_act call
__global__ void int_threshold_kernel(const __half* __restrict__ bias, const __half* __restrict__ bias_noise,
                                     int32_t* __restrict__ out, int64_t P, int64_t N, int offset) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= P * N) return;
  out[e] = __half2int_rz(__hadd(bias[e % N], bias_noise[e])) + offset;
}

// ---- set_noise ---------------------------------------------------------------------------------------
// P = half(sigmoid(float(half(half(w / m1) * 5)))), m1 = half(half(mean |w|) + 1e-5)
__global__ void __launch_bounds__(1024) abs_sum_kernel(const __half* __restrict__ w, float* __restrict__ sum, int64_t n) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    acc += fabsf(__half2float(w[i]));
#pragma unroll
  for (int sh = 16; sh > 0; sh >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sh);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
    if (threadIdx.x == 0) atomicAdd(sum, v);
  }
}

__global__ void probabilities_kernel(const __half* __restrict__ w, const float* __restrict__ sum, __half* __restrict__ p, int64_t n) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const __half mean = __float2half_rn(*sum / float(n));
  const __half m1 = __float2half_rn(__half2float(mean) + 1e-5f);
  const __half q = __float2half_rn(__half2float(w[i]) / __half2float(m1));
  const __half q5 = __float2half_rn(__half2float(q) * 5.f);
  p[i] = __float2half_rn(1.f / (1.f + expf(-__half2float(q5))));
}

// bias noise: half(half(u - 0.5) * 6) with u a half uniform in [0, 1)
__global__ void bias_noise_kernel(__half* __restrict__ out, int64_t n, uint64_t seed, uint64_t offset) {
  const int64_t q = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (q * 4 >= n) return;
  const uint64_t ctr = offset + uint64_t(q);
  uint32_t r[4];
  Philox ph(seed);
  ph(uint32_t(ctr), uint32_t(ctr >> 32), 0u, 6u, r);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (q * 4 + j < n) {
      const __half u = __float2half_rn(float(r[j] >> 21) * (1.0f / 2048.0f));      // 11 random bits: every half in [0, 1) on that grid
      const __half c = __hsub(u, __float2half_rn(0.5f));
      out[q * 4 + j] = __float2half_rn(__half2float(c) * 6.f);
    }
}

// ---- update ------------------------------------------------------------------------------------------
// w_h[d] = half(half(f[d]) - half(mean over d of half(f[d])))      (one block)
__global__ void __launch_bounds__(1024) centre_fitness_kernel(const float* __restrict__ f, __half* __restrict__ out, int64_t D) {
  __shared__ float red[32];
  __shared__ float mean_s;
  float acc = 0.f;
  for (int64_t d = threadIdx.x; d < D; d += blockDim.x) acc += __half2float(__float2half_rn(f[d]));
#pragma unroll
  for (int sh = 16; sh > 0; sh >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sh);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = red[threadIdx.x];
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
    if (threadIdx.x == 0) mean_s = __half2float(__float2half_rn(v / float(D)));
  }
  __syncthreads();
  const __half mean = __float2half_rn(mean_s);
  for (int64_t d = threadIdx.x; d < D; d += blockDim.x) out[d] = __hsub(__float2half_rn(f[d]), mean);
}

// grad = half(half(grad + half(l1 * sign(W))) + half(l2 * W))
__global__ void regularise_half_kernel(__half* __restrict__ grad, const __half* __restrict__ weight, int64_t n, float l1, float l2) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float wv = __half2float(weight[i]);
  __half g = grad[i];
  if (l1 != 0.f) g = __hadd(g, __float2half_rn(l1 * float((wv > 0.f) - (wv < 0.f))));
  if (l2 != 0.f) g = __hadd(g, __float2half_rn(l2 * wv));
  grad[i] = g;
}

// bias_grad[m] = half(sum_d float(w_h[d]) * float(bias_noise[d, m]))
__global__ void __launch_bounds__(256) bias_grad_half_kernel(const __half* __restrict__ w, const __half* __restrict__ bn,
                                                             __half* __restrict__ out, int64_t D, int64_t N) {
  __shared__ float red[256];
  const int t = threadIdx.x, lane = t & 31, grp = t >> 5;
  const int64_t n = int64_t(blockIdx.x) * 32 + lane;
  float acc = 0.f;
  if (n < N) {
#pragma unroll 4
    for (int64_t d = grp; d < D; d += 8) acc = fmaf(__half2float(w[d]), __half2float(bn[d * N + n]), acc);
  }
  red[t] = acc;
  __syncthreads();
  if (t < 32 && n < N) {
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) s += red[u * 32 + t];
    out[n] = __float2half_rn(s);
  }
}

template <int MODE>
static int launch_bmv_rows(const void* A, const void* X, void* out, const __half* bias, const __half* bn, int64_t P, int64_t M,
                           int cpr, int n_bits, int64_t out_row_u32, cudaStream_t st) {
  const int64_t gpm = ceil_div<int64_t>(M, 32), groups = gpm * P;
  const int64_t want = ceil_div<int64_t>(groups, 16);              // two groups per warp and pass at least
  const int64_t cap = int64_t(sm_count()) * 4;
  const unsigned grid = (unsigned)(want < cap ? (want > 0 ? want : 1) : cap);
  const uint4* a = static_cast<const uint4*>(A);
  const uint4* x = static_cast<const uint4*>(X);
  if (cpr <= 4) bmv_rows_kernel<MODE, 4, 1><<<grid, 256, 0, st>>>(a, x, out, bias, bn, M, cpr, n_bits, out_row_u32, gpm, groups);
  else if (cpr <= 8) bmv_rows_kernel<MODE, 8, 1><<<grid, 256, 0, st>>>(a, x, out, bias, bn, M, cpr, n_bits, out_row_u32, gpm, groups);
  else if (cpr <= 16) bmv_rows_kernel<MODE, 8, 2><<<grid, 256, 0, st>>>(a, x, out, bias, bn, M, cpr, n_bits, out_row_u32, gpm, groups);
  else bmv_rows_kernel<MODE, 8, 4><<<grid, 256, 0, st>>>(a, x, out, bias, bn, M, cpr, n_bits, out_row_u32, gpm, groups);
  return check_launch("binarized_linear_fwd");
}

// true when the row-streaming product covers the shape: rows are whole 16-byte chunks, at most 32 of them
bool bmv_rows_covers(const void* A, const void* X, int64_t P, int64_t K, int word_bits) {
  const int64_t row_bytes = K * (word_bits / 8);
  (void)P;
  return K > 0 && row_bytes % 16 == 0 && row_bytes / 16 <= 32 && aligned16(A) && aligned16(X);
}

int bmv_rows_counts(const void* A, const void* X, int32_t* counts, int64_t P, int64_t M, int64_t K, int word_bits, cudaStream_t st) {
  return launch_bmv_rows<BMV_COUNTS>(A, X, counts, nullptr, nullptr, P, M, int(K * (word_bits / 8) / 16), 0, 0, st);
}

}  // namespace nes

using namespace nes;

extern "C" int nes_binarized_probabilities(const uint16_t* weight_half, uint16_t* p_half, float* scratch_sum, int64_t n,
                                           nes_stream_t stream) {
  NES_REQUIRE(n >= 0, NES_ERR_BAD_ARG, "binarized_probabilities: negative extent");
  if (n == 0) return NES_OK;
  NES_REQUIRE(weight_half && p_half && scratch_sum, NES_ERR_BAD_ARG, "binarized_probabilities: null pointer");
  cudaStream_t st = as_stream(stream);
  cudaMemsetAsync(scratch_sum, 0, sizeof(float), st);
  const int64_t want = ceil_div<int64_t>(n, 1024);
  const unsigned blocks = (unsigned)(want < 1024 ? want : 1024);
  abs_sum_kernel<<<blocks, 1024, 0, st>>>(reinterpret_cast<const __half*>(weight_half), scratch_sum, n);
  int rc = check_launch("binarized_probabilities(mean)");
  if (rc != NES_OK) return rc;
  probabilities_kernel<<<(unsigned)ceil_div<int64_t>(n, 256), 256, 0, st>>>(reinterpret_cast<const __half*>(weight_half), scratch_sum,
                                                                           reinterpret_cast<__half*>(p_half), n);
  return check_launch("binarized_probabilities");
}

extern "C" int nes_binarized_bias_noise(uint16_t* out_half, int64_t n, uint64_t seed, uint64_t offset, nes_stream_t stream) {
  NES_REQUIRE(n >= 0, NES_ERR_BAD_ARG, "binarized_bias_noise: negative extent");
  if (n == 0) return NES_OK;
  NES_REQUIRE(out_half, NES_ERR_BAD_ARG, "binarized_bias_noise: null pointer");
  const int64_t groups = ceil_div<int64_t>(n, 4);
  bias_noise_kernel<<<(unsigned)ceil_div<int64_t>(groups, 256), 256, 0, as_stream(stream)>>>(reinterpret_cast<__half*>(out_half), n, seed, offset);
  return check_launch("binarized_bias_noise");
}

extern "C" int64_t nes_binarized_update_scratch_bytes(int64_t D, int64_t rows, int64_t words, int word_bits) {
  return nes_bin_weighted_sum_scratch_bytes(D, rows, words, word_bits) + ((D * 2 + 255) & ~int64_t(255));
}

extern "C" int nes_binarized_update(const void* noise_bits, const float* fitness, const uint16_t* weight_half,
                                    const uint16_t* bias_noise_half, uint16_t* grad_half, uint16_t* bias_grad_half,
                                    int64_t D, int64_t rows, int64_t words, int64_t zbits, int64_t out_degree, int word_bits,
                                    float l1, float l2, void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  NES_REQUIRE(D > 0 && rows >= 0 && words >= 0 && zbits >= 0 && out_degree >= 0, NES_ERR_BAD_ARG, "binarized_update: bad extent");
  NES_REQUIRE(noise_bits && fitness && grad_half, NES_ERR_BAD_ARG, "binarized_update: null pointer");
  NES_REQUIRE((l1 == 0.f && l2 == 0.f) || weight_half, NES_ERR_BAD_ARG, "binarized_update: l1/l2 given without weight");
  NES_REQUIRE((bias_noise_half == nullptr) == (bias_grad_half == nullptr), NES_ERR_BAD_ARG,
              "binarized_update: bias_noise and bias_grad go together");
  const int64_t need = nes_binarized_update_scratch_bytes(D, rows, words, word_bits);
  NES_REQUIRE(scratch && scratch_bytes >= need && aligned16(scratch), NES_ERR_SCRATCH,
              "binarized_update: scratch needs %lld bytes, 16-byte aligned", (long long)need);
  cudaStream_t st = as_stream(stream);
  const int64_t w_bytes = (D * 2 + 255) & ~int64_t(255);
  __half* w_h = static_cast<__half*>(scratch);
  centre_fitness_kernel<<<1, 1024, 0, st>>>(fitness, w_h, D);
  int rc = check_launch("binarized_update(centre)");
  if (rc != NES_OK) return rc;
  rc = bin_weighted_sum_impl(noise_bits, reinterpret_cast<const uint16_t*>(w_h), grad_half, D, rows, words, zbits, word_bits,
                             static_cast<unsigned char*>(scratch) + w_bytes, scratch_bytes - w_bytes, st);
  if (rc != NES_OK) return rc;
  const int64_t n = rows * zbits;
  if ((l1 != 0.f || l2 != 0.f) && n > 0) {
    regularise_half_kernel<<<(unsigned)ceil_div<int64_t>(n, 256), 256, 0, st>>>(reinterpret_cast<__half*>(grad_half),
                                                                               reinterpret_cast<const __half*>(weight_half), n, l1, l2);
    if ((rc = check_launch("binarized_update(l1/l2)")) != NES_OK) return rc;
  }
  if (bias_grad_half && out_degree > 0) {
    bias_grad_half_kernel<<<(unsigned)ceil_div<int64_t>(out_degree, 32), 256, 0, st>>>(
        w_h, reinterpret_cast<const __half*>(bias_noise_half), reinterpret_cast<__half*>(bias_grad_half), D, out_degree);
    if ((rc = check_launch("binarized_update(bias)")) != NES_OK) return rc;
  }
  return NES_OK;
}

// out_kind: 0 activation int32 (2 * counts - in_bits), 1 bool bytes, 2 bits packed along the output rows
extern "C" int64_t nes_binarized_linear_fwd_scratch_bytes(int64_t D, int64_t out, int batch_norm) {
  return batch_norm ? (D * out * 4 + ((out * 4 + 255) & ~int64_t(255))) : 0;
}

extern "C" int nes_binarized_linear_fwd(const void* weight_bits, const void* x_packed, const uint16_t* bias_half,
                                        const uint16_t* bias_noise_half, void* out, int64_t D, int64_t out_f, int64_t words,
                                        int in_bits, int word_bits, int out_kind, int batch_norm,
                                        void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && out_f >= 0 && words > 0 && in_bits >= 0, NES_ERR_BAD_ARG, "binarized_linear_fwd: bad extent");
  NES_REQUIRE(word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "binarized_linear_fwd: word_bits must be 32 or 64");
  NES_REQUIRE(out_kind >= 0 && out_kind <= 2, NES_ERR_BAD_ARG, "binarized_linear_fwd: out_kind must be 0, 1 or 2");
  if (D == 0 || out_f == 0) return NES_OK;
  NES_REQUIRE(weight_bits && x_packed && out, NES_ERR_BAD_ARG, "binarized_linear_fwd: null pointer");
  NES_REQUIRE(out_kind == 0 || (bias_half && bias_noise_half), NES_ERR_BAD_ARG, "binarized_linear_fwd: thresholds need bias and bias_noise");
  NES_REQUIRE(bmv_rows_covers(weight_bits, x_packed, D, words, word_bits), NES_ERR_UNSUPPORTED,
              "binarized_linear_fwd: rows must be whole 16-byte chunks (at most 32), operands 16-byte aligned, D <= 65535");
  cudaStream_t st = as_stream(stream);
  const int cpr = int(words * (word_bits / 8) / 16);
  const __half* bias = reinterpret_cast<const __half*>(bias_half);
  const __half* bn = reinterpret_cast<const __half*>(bias_noise_half);
  const int64_t out_row_u32 = ceil_div<int64_t>(out_f, word_bits) * (word_bits / 32);
  if (out_kind == 2 && out_row_u32 * 32 != ((out_f + 31) & ~int64_t(31)))
    cudaMemsetAsync(out, 0, D * out_row_u32 * 4, st);          // a trailing 32-bit half of the last int64 word stays zero
  if (out_kind == 0) return launch_bmv_rows<BMV_ACT>(weight_bits, x_packed, out, nullptr, nullptr, D, out_f, cpr, in_bits, 0, st);
  if (!batch_norm) {
    if (out_kind == 1) return launch_bmv_rows<BMV_BOOL>(weight_bits, x_packed, out, bias, bn, D, out_f, cpr, in_bits, 0, st);
    return launch_bmv_rows<BMV_PACKED>(weight_bits, x_packed, out, bias, bn, D, out_f, cpr, in_bits, out_row_u32, st);
  }
  // batch mean over the members: activations, their column sums, then the compare
  const int64_t need = nes_binarized_linear_fwd_scratch_bytes(D, out_f, 1);
  NES_REQUIRE(scratch && scratch_bytes >= need && aligned16(scratch), NES_ERR_SCRATCH,
              "binarized_linear_fwd: scratch needs %lld bytes, 16-byte aligned", (long long)need);
  float* sums = static_cast<float*>(scratch);
  int32_t* act = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(scratch) + ((out_f * 4 + 255) & ~int64_t(255)));
  int rc = launch_bmv_rows<BMV_ACT>(weight_bits, x_packed, act, nullptr, nullptr, D, out_f, cpr, in_bits, 0, st);
  if (rc != NES_OK) return rc;
  act_colsum_kernel<<<dim3((unsigned)ceil_div<int64_t>(out_f, 32), 1), 256, 0, st>>>(act, sums, D, 1, out_f, 0, 0, 1);
  if ((rc = check_launch("binarized_linear_fwd(mean)")) != NES_OK) return rc;
  const int64_t warps = D * ceil_div<int64_t>(out_f, 32);
  const unsigned blocks = (unsigned)ceil_div<int64_t>(warps * 32, 256);
  if (out_kind == 1)
    act_threshold_kernel<false><<<blocks, 256, 0, st>>>(act, bias, bn, sums, out, D, 1, out_f, 0, 0, 1, float(D), 0);
  else
    act_threshold_kernel<true><<<blocks, 256, 0, st>>>(act, bias, bn, sums, out, D, 1, out_f, 0, 0, 1, float(D), out_row_u32);
  return check_launch("binarized_linear_fwd(threshold)");
}

// Epilogue of BinarizedConv2d on the counts of nes_bin_conv, counts (P, S, N) with S = h * w positions:
// act = 2 * counts - offset; out_kind 0: act int32; 1 / 2: half(act) > half(bias + bias_noise + mean over the
// member's positions of half(act)) as bool bytes / as bits packed along the channels (the layout the next
// packed NHWC layer reads).  sums: P * N floats of scratch (batch_norm only).
extern "C" int nes_binarized_conv_epilogue(const int32_t* counts, const uint16_t* bias_half, const uint16_t* bias_noise_half,
                                           void* out, int64_t P, int64_t S, int64_t N, int offset, int word_bits,
                                           int out_kind, int batch_norm, float* sums, nes_stream_t stream) {
  NES_REQUIRE(P >= 0 && S >= 0 && N >= 0, NES_ERR_BAD_ARG, "binarized_conv_epilogue: negative extent");
  NES_REQUIRE(out_kind >= 0 && out_kind <= 2 && (word_bits == 32 || word_bits == 64), NES_ERR_BAD_ARG, "binarized_conv_epilogue: bad option");
  if (P * S * N == 0) return NES_OK;
  NES_REQUIRE(counts && out, NES_ERR_BAD_ARG, "binarized_conv_epilogue: null pointer");
  cudaStream_t st = as_stream(stream);
  const int64_t warps = P * S * ceil_div<int64_t>(N, 32);
  NES_REQUIRE(ceil_div<int64_t>(warps * 32, 256) <= INT32_MAX && P <= 65535, NES_ERR_UNSUPPORTED, "binarized_conv_epilogue: too large");
  const unsigned blocks = (unsigned)ceil_div<int64_t>(warps * 32, 256);
  if (out_kind == 0) {
    const int64_t n = P * S * N;
    act_from_counts_kernel<<<(unsigned)ceil_div<int64_t>(n, 256), 256, 0, st>>>(counts, static_cast<int32_t*>(out), n, offset);
    return check_launch("binarized_conv_epilogue(activation)");
  }
  NES_REQUIRE(bias_half && bias_noise_half, NES_ERR_BAD_ARG, "binarized_conv_epilogue: thresholds need bias and bias_noise");
  const __half* bias = reinterpret_cast<const __half*>(bias_half);
  const __half* bn = reinterpret_cast<const __half*>(bias_noise_half);
  if (batch_norm) {
    NES_REQUIRE(sums, NES_ERR_SCRATCH, "binarized_conv_epilogue: the batch mean needs P * N floats of scratch");
    act_colsum_kernel<<<dim3((unsigned)ceil_div<int64_t>(N, 32), (unsigned)P), 256, 0, st>>>(counts, sums, P, S, N, 1, offset, 0);
    int rc = check_launch("binarized_conv_epilogue(mean)");
    if (rc != NES_OK) return rc;
  }
  const int64_t out_row_u32 = ceil_div<int64_t>(N, word_bits) * (word_bits / 32);
  if (out_kind == 2 && out_row_u32 * 32 != ((N + 31) & ~int64_t(31))) cudaMemsetAsync(out, 0, P * S * out_row_u32 * 4, st);
  if (out_kind == 1)
    act_threshold_kernel<false><<<blocks, 256, 0, st>>>(counts, bias, bn, batch_norm ? sums : nullptr, out, P, S, N, 1, offset, 0, float(S), 0);
  else
    act_threshold_kernel<true><<<blocks, 256, 0, st>>>(counts, bias, bn, batch_norm ? sums : nullptr, out, P, S, N, 1, offset, 0, float(S), out_row_u32);
  return check_launch("binarized_conv_epilogue");
}

extern "C" int nes_binarized_int_threshold(const uint16_t* bias_half, const uint16_t* bias_noise_half, int32_t* out,
                                           int64_t P, int64_t N, int offset, nes_stream_t stream) {
  NES_REQUIRE(P >= 0 && N >= 0, NES_ERR_BAD_ARG, "binarized_int_threshold: negative extent");
  if (P * N == 0) return NES_OK;
  NES_REQUIRE(bias_half && bias_noise_half && out, NES_ERR_BAD_ARG, "binarized_int_threshold: null pointer");
  int_threshold_kernel<<<(unsigned)ceil_div<int64_t>(P * N, 256), 256, 0, as_stream(stream)>>>(
      reinterpret_cast<const __half*>(bias_half), reinterpret_cast<const __half*>(bias_noise_half), out, P, N, offset);
  return check_launch("binarized_int_threshold");
}
