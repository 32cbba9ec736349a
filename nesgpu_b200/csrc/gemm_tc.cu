// Tensor-core GEMM for sm_100a: C[M,N] = A[M,K] . B[N,K]^T (+ bias), fp32 in / fp32 out.
//
// Blackwell execution model, written directly in PTX:
//   * operands travel global -> shared memory as 128-byte-swizzled tiles by TMA
//     (cp.async.bulk.tensor.2d, one elected producer thread, mbarrier transaction counts);
//   * one warp runs the MMA loop in converged control flow and an elected lane issues tcgen05.mma
//     (kind::tf32, M = 128, N = 128, K = 8 per instruction) with both operands read from shared memory
//     through matrix descriptors and the fp32 accumulator tile (128 lanes x 128 columns) living in
//     tensor memory;
//   * tcgen05.commit hands shared-memory stages back to the producer and signals the epilogue;
//   * four epilogue warps read the accumulator with tcgen05.ld (one TMEM lane = one output
//     row per thread), add the bias and store.
// With BF16 the operands are bf16 (64 elements per 128-byte row, kind::f16 with K = 16); TERMS = 3 with BF16 is the
// split-bf16 form: the same three products on bf16 hi / lo parts, half the operand bytes of 3xTF32.
// Precision modes: TERMS = 1 is plain TF32 (inputs rounded to 10 mantissa bits; relative error
// ~1e-3, for callers that state it).  TERMS = 3 is the error-compensated 3xTF32 scheme: every
// operand is split beforehand into hi = tf32(a) and lo = a - hi, and the kernel accumulates
// a_lo.b_hi + a_hi.b_lo + a_hi.b_hi, which keeps fp32-level accuracy (~1e-6) on the tensor pipe.
//
// Every wait on an mbarrier is bounded: when the limit is hit the thread records an error code
// in a device word (read by nes_tc_error_flag), stops issuing work and falls through to the
// common exit, where tensor memory is released.
#include <cuda_bf16.h>
#include "tc_ptx.cuh"

namespace nes {
namespace tc {

constexpr int BM = 128, BN = 128, BKE = 32;          // tile, K elements (fp32) per stage = one 128-byte swizzle row
constexpr int TILE_BYTES = BM * BKE * 4;             // 16 KiB per operand tile
constexpr int NTHREADS = 192;                        // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue

struct Maps { CUtensorMap a_hi, b_hi, a_lo, b_lo; };

// Optional per-row epilogue term of the population-batched layers: row gm belongs to member gm % D and
// repeat gm / D, and receives sign(repeat) * bias_noise[member, column].
struct RowTerm { const float* bias_noise; int64_t D, R; int antithetic; };

template <int TERMS, bool BF16 = false>
__global__ void __launch_bounds__(NTHREADS, 1) gemm_tf32_kernel(const __grid_constant__ Maps maps, const float* __restrict__ bias,
                                                                 const RowTerm rt, float* __restrict__ C, int M, int N, int K, int stages) {
  extern __shared__ unsigned char dyn_raw[];
  const unsigned int timeouts_at_start = timeouts_so_far();
  constexpr int OPERANDS = (TERMS == 3) ? 4 : 2;
  constexpr int STAGE_BYTES = OPERANDS * TILE_BYTES;
  // 1 KiB-aligned tile area, then the barriers
  const uint32_t raw = smem_u32(dyn_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  unsigned char* tiles = dyn_raw + pad;
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + size_t(stages) * STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* accum = empty + stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  constexpr int BKS = BF16 ? 2 * BKE : BKE;          // K elements per stage (one 128-byte row)
  const int nk = (K + BKS - 1) / BKS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(accum, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: one TMA load per operand tile and stage
      for (int kt = 0; kt < nk; ++kt) {
        const int s = kt % stages;
        const uint32_t ph = (kt / stages) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, 1)) break;
        unsigned char* st = tiles + size_t(s) * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        tma_load_2d(st, &maps.a_hi, &full[s], kt * BKS, m0);
        tma_load_2d(st + TILE_BYTES, &maps.b_hi, &full[s], kt * BKS, n0);
        if (TERMS == 3) {
          tma_load_2d(st + 2 * TILE_BYTES, &maps.a_lo, &full[s], kt * BKS, m0);
          tma_load_2d(st + 3 * TILE_BYTES, &maps.b_lo, &full[s], kt * BKS, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the whole warp runs this loop in converged control flow, one elected lane issues
    constexpr uint32_t idesc = BF16 ? idesc_bf16(BM, BN) : idesc_tf32(BM, BN);
    // descriptors are a constant plus an offset in 16-byte units: the stage's tiles lie TILE_BYTES apart
    const uint64_t desc0 = smem_desc_sw128(smem_u32(tiles));
    constexpr uint32_t TILE_UNITS = TILE_BYTES >> 4;
    bool ok = true;
    int s = 0;
    uint32_t ph = 0;
    for (int kt = 0; kt < nk && ok; ++kt) {
      ok = warp_mbar_wait(&full[s], ph, 2);
      if (!ok) break;
      tc_fence_after();
      const uint64_t a_hi = desc0 + uint64_t(uint32_t(s) * uint32_t(STAGE_BYTES >> 4));
      const uint64_t b_hi = a_hi + TILE_UNITS;
#pragma unroll
      for (int k = 0; k < BKE / 8; ++k) {            // advance 32 bytes (2 descriptor units) per K = 8
        const uint64_t adv = uint64_t(k * 2);
        if (TERMS == 3) {
          const uint64_t a_lo = a_hi + 2 * TILE_UNITS, b_lo = a_hi + 3 * TILE_UNITS;
          if (BF16) {
            warp_mma_bf16(tmem_base, a_lo + adv, b_hi + adv, idesc, (kt > 0 || k > 0) ? 1u : 0u);
            warp_mma_bf16(tmem_base, a_hi + adv, b_lo + adv, idesc, 1u);
            warp_mma_bf16(tmem_base, a_hi + adv, b_hi + adv, idesc, 1u);
          } else {
            warp_mma_tf32(tmem_base, a_lo + adv, b_hi + adv, idesc, (kt > 0 || k > 0) ? 1u : 0u);
            warp_mma_tf32(tmem_base, a_hi + adv, b_lo + adv, idesc, 1u);
            warp_mma_tf32(tmem_base, a_hi + adv, b_hi + adv, idesc, 1u);
          }
        } else if (BF16) {
          warp_mma_bf16(tmem_base, a_hi + adv, b_hi + adv, idesc, (kt > 0 || k > 0) ? 1u : 0u);
        } else {
          warp_mma_tf32(tmem_base, a_hi + adv, b_hi + adv, idesc, (kt > 0 || k > 0) ? 1u : 0u);
        }
      }
      warp_mma_commit(&empty[s]);            // frees the stage once these MMAs have read it
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
    warp_mma_commit(accum);                  // accumulator complete (or abandoned: epilogue checks the error word)
  } else {
    // ---- epilogue: warp w may touch TMEM lanes 32*(w%4) .. +31
    const int q = warp & 3;
    const bool ok = mbar_wait_relaxed(accum, 0, 3);
    tc_fence_after();
    if (ok && timeouts_so_far() == timeouts_at_start && nk > 0) {
      const int64_t gm = int64_t(m0) + q * 32 + lane;
      const float* bn_row = nullptr;
      float bn_sign = 1.f;
      if (rt.bias_noise && gm < M) {
        bn_row = rt.bias_noise + (gm % rt.D) * N;
        bn_sign = anti_sign(gm / rt.D, rt.R, rt.antithetic);
      }
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(c), r);
        if (gm < M) {
          float* dst = C + gm * N + n0 + c;
          const bool vec = ((N & 3) == 0);
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int gn = n0 + c + j;
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              v[u] = __uint_as_float(r[j + u]);
              if (bias && gn + u < N) v[u] += __ldg(bias + gn + u);
              if (bn_row && gn + u < N) v[u] += bn_sign * __ldg(bn_row + gn + u);
            }
            if (vec && gn + 3 < N) {
              *reinterpret_cast<float4*>(dst + j) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
#pragma unroll
              for (int u = 0; u < 4; ++u) if (gn + u < N) dst[j + u] = v[u];
            }
          }
        }
      }
    } else if (ok && nk == 0) {
      const int64_t gm = int64_t(m0) + q * 32 + lane;
      if (gm < M)
        for (int j = 0; j < BN; ++j)
          if (n0 + j < N) {
            float v = bias ? bias[n0 + j] : 0.f;
            if (rt.bias_noise) v += anti_sign(gm / rt.D, rt.R, rt.antithetic) * rt.bias_noise[(gm % rt.D) * N + n0 + j];
            C[gm * N + n0 + j] = v;
          }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, BN);
  }
}

// hi = a rounded to tf32 (10 mantissa bits, round to nearest even), lo = a - hi
__global__ void split_tf32_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo, int64_t n) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float a = src[i];
  const float h = round_tf32(a);
  hi[i] = h;
  if (lo) lo[i] = a - h;
}

// Operand of the permuted layer's single product: row b of A2 is [ x[b, :] | s(b) * x[b, pin[d, :]] | 0.. ],
// rounded to tf32 (hi) with the residual kept (lo) for the 3-term scheme.  One block per row; the row is
// read once coalesced, the gather then hits it in L1/L2.
template <bool BF16>
__global__ void __launch_bounds__(256) permuted_operand_kernel(const float* __restrict__ x, const int16_t* __restrict__ pin,
                                                               float* __restrict__ hi, float* __restrict__ lo,
                                                               int64_t B, int64_t D, int64_t R, int in, int in_sp, int K2,
                                                               int antithetic) {
  // a thread produces four consecutive columns and stores them with one instruction per array; with
  // in and in_sp multiples of 4 (and 16-byte aligned x) the plain part and the permutation are read as vectors
  const bool vec = (in % 4 == 0) && (in_sp % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
                   (pin == nullptr || (reinterpret_cast<uintptr_t>(pin) & 7u) == 0);
  for (int64_t b = blockIdx.x; b < B; b += gridDim.x) {
    const int64_t d = b % D;
    const float sgn = anti_sign(b / D, R, antithetic);
    const float* xr = x + b * in;
    const int16_t* pr = pin ? pin + d * in_sp : nullptr;
    for (int k0 = threadIdx.x * 4; k0 < K2; k0 += blockDim.x * 4) {
      float a[4];
      if (vec && k0 + 3 < in) {
        const float4 v = *reinterpret_cast<const float4*>(xr + k0);
        a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
      } else if (vec && k0 >= in && k0 + 3 < in + in_sp) {
        int j[4];
        if (pr) {
          const short4 pv = *reinterpret_cast<const short4*>(pr + (k0 - in));
          j[0] = pv.x; j[1] = pv.y; j[2] = pv.z; j[3] = pv.w;
        } else {
          j[0] = k0 - in; j[1] = j[0] + 1; j[2] = j[0] + 2; j[3] = j[0] + 3;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) a[u] = sgn * xr[j[u]];
      } else {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int k = k0 + u;
          a[u] = 0.f;
          if (k < in) a[u] = xr[k];
          else if (k < in + in_sp) a[u] = sgn * xr[pr ? int(pr[k - in]) : k - in];
        }
      }
      if (BF16) {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(a[0], a[1]), p1 = __floats2bfloat162_rn(a[2], a[3]);
        uint2 w;
        w.x = *reinterpret_cast<uint32_t*>(&p0);
        w.y = *reinterpret_cast<uint32_t*>(&p1);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(hi) + b * K2 + k0) = w;
        if (lo) {                  // split form: what the bf16 rounding left over, again as bf16
          p0 = __floats2bfloat162_rn(a[0] - __uint_as_float(w.x << 16), a[1] - __uint_as_float(w.x & 0xffff0000u));
          p1 = __floats2bfloat162_rn(a[2] - __uint_as_float(w.y << 16), a[3] - __uint_as_float(w.y & 0xffff0000u));
          w.x = *reinterpret_cast<uint32_t*>(&p0);
          w.y = *reinterpret_cast<uint32_t*>(&p1);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(lo) + b * K2 + k0) = w;
        }
      } else {
        float h[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) h[u] = round_tf32(a[u]);
        *reinterpret_cast<float4*>(hi + b * K2 + k0) = make_float4(h[0], h[1], h[2], h[3]);
        if (lo) *reinterpret_cast<float4*>(lo + b * K2 + k0) = make_float4(a[0] - h[0], a[1] - h[1], a[2] - h[2], a[3] - h[3]);
      }
    }
  }
}

// B2[o, :] = [ weight[o, :] | eps[o, :] (rows below out_sp, else 0) | 0.. ]
template <bool BF16>
__global__ void permuted_filter_kernel(const float* __restrict__ w, const float* __restrict__ eps,
                                       float* __restrict__ hi, float* __restrict__ lo, int64_t out, int64_t out_sp,
                                       int in, int in_sp, int K2) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= out * K2) return;
  const int64_t o = i / K2;
  const int k = int(i - o * K2);
  float a = 0.f;
  if (k < in) a = w[o * in + k];
  else if (k < in + in_sp && o < out_sp) a = eps[o * in_sp + (k - in)];
  if (BF16) {
    const __nv_bfloat16 h = __float2bfloat16_rn(a);
    reinterpret_cast<__nv_bfloat16*>(hi)[i] = h;
    if (lo) reinterpret_cast<__nv_bfloat16*>(lo)[i] = __float2bfloat16_rn(a - __bfloat162float(h));
  } else {
    const float h = round_tf32(a);
    hi[i] = h;
    if (lo) lo[i] = a - h;
  }
}

// hi / lo split of x[b, :] * flips[b % D, :] (sign-flip sampling: the noise product's A operand)
__global__ void split_flipped_kernel(const float* __restrict__ x, const int8_t* __restrict__ flips, float* __restrict__ hi,
                                     float* __restrict__ lo, int64_t B, int64_t D, int64_t in) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= B * in) return;
  const int64_t b = i / in, c = i - b * in;
  const float a = x[i] * float(flips[(b % D) * in + c]);
  const float h = round_tf32(a);
  hi[i] = h;
  if (lo) lo[i] = a - h;
}

// y[b, o] += s(r) * (p[b, o] * fout[d, o] + beta[d, o])        (sign-flip sampling, modules/base.py:620-626)
__global__ void synthetic_combine_kernel(float* __restrict__ y, const float* __restrict__ p, const int8_t* __restrict__ fout,
                                         const float* __restrict__ beta, int64_t B, int64_t D, int64_t R, int64_t out,
                                         int antithetic) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= B * out) return;
  const int64_t b = i / out, o = i - b * out;
  const int64_t d = b % D;
  float q = p[i];
  if (fout) q *= float(fout[d * out + o]);
  if (beta) q += __ldg(beta + d * out + o);
  y[i] += anti_sign(b / D, R, antithetic) * q;
}

// y[b, o] += s(r) * (sum_t x[b, idx[d, o, t]] * val[d, o, t] + beta[d, o])     (sparse per-member noise)
__global__ void sparse_noise_add_kernel(float* __restrict__ y, const float* __restrict__ x, const int32_t* __restrict__ idx,
                                        const float* __restrict__ val, const float* __restrict__ beta, int64_t B, int64_t D,
                                        int64_t R, int64_t in, int64_t out, int k, int antithetic) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= B * out) return;
  const int64_t b = i / out, o = i - b * out;
  const int64_t d = b % D;
  const int64_t e = (d * out + o) * k;
  const float* xr = x + b * in;
  float q = 0.f;
  for (int t = 0; t < k; ++t) q = fmaf(__ldg(xr + idx[e + t]), __ldg(val + e + t), q);
  if (beta) q += __ldg(beta + d * out + o);
  y[i] += anti_sign(b / D, R, antithetic) * q;
}

// 2-D fp32 row-major [rows][cols] tensor, box = 32 columns x box_rows rows, 128-byte swizzle, zero fill
static int make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int box_rows, const char* what,
                    bool bf16 = false) {
  EncodeTiledFn fn = encode_fn();
  NES_REQUIRE(fn != nullptr, NES_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", what);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * (bf16 ? 2 : 4)};
  cuuint32_t box[2] = {(cuuint32_t)(bf16 ? 2 * BKE : BKE), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NES_REQUIRE(r == CUDA_SUCCESS, NES_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
  return NES_OK;
}

static int64_t align256(int64_t v) { return (v + 255) & ~int64_t(255); }

// Launches the tile kernel on prepared (rounded / split) operands.
static int run_gemm(const float* a_hi, const float* a_lo, const float* b_hi, const float* b_lo, const float* bias,
                    const RowTerm& rt, float* y, int64_t M, int64_t N, int64_t K, int mode, cudaStream_t st, const char* what) {
  int rc;
  Maps maps;
  // modes: 1 TF32, 2 bf16, 3 3xTF32 (tf32 hi / lo splits), 4 split-bf16 (bf16 hi / lo splits, three products)
  const bool bf16 = (mode == 2 || mode == 4);
  const bool three = (mode == 3 || mode == 4);
  if ((rc = make_map(&maps.a_hi, a_hi, M, K, BM, what, bf16)) != NES_OK) return rc;
  if ((rc = make_map(&maps.b_hi, b_hi, N, K, BN, what, bf16)) != NES_OK) return rc;
  if (three) {
    if ((rc = make_map(&maps.a_lo, a_lo, M, K, BM, what, bf16)) != NES_OK) return rc;
    if ((rc = make_map(&maps.b_lo, b_lo, N, K, BN, what, bf16)) != NES_OK) return rc;
  } else {
    maps.a_lo = maps.a_hi;
    maps.b_lo = maps.b_hi;
  }
  const int stages = three ? 3 : 4;
  const int stage_bytes = (three ? 4 : 2) * TILE_BYTES;
  const size_t smem = 1024 + size_t(stages) * stage_bytes + (2 * stages + 1) * sizeof(uint64_t) + 16;
  dim3 grid((unsigned)ceil_div<int64_t>(M, BM), (unsigned)ceil_div<int64_t>(N, BN));
  cudaError_t e;
  if (mode == 4) {
    e = cudaFuncSetAttribute(gemm_tf32_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "%s: shared memory opt-in failed: %s", what, cudaGetErrorString(e));
    gemm_tf32_kernel<3, true><<<grid, NTHREADS, smem, st>>>(maps, bias, rt, y, int(M), int(N), int(K), stages);
  } else if (mode == 3) {
    e = cudaFuncSetAttribute(gemm_tf32_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "%s: shared memory opt-in failed: %s", what, cudaGetErrorString(e));
    gemm_tf32_kernel<3><<<grid, NTHREADS, smem, st>>>(maps, bias, rt, y, int(M), int(N), int(K), stages);
  } else if (bf16) {
    e = cudaFuncSetAttribute(gemm_tf32_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "%s: shared memory opt-in failed: %s", what, cudaGetErrorString(e));
    gemm_tf32_kernel<1, true><<<grid, NTHREADS, smem, st>>>(maps, bias, rt, y, int(M), int(N), int(K), stages);
  } else {
    e = cudaFuncSetAttribute(gemm_tf32_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "%s: shared memory opt-in failed: %s", what, cudaGetErrorString(e));
    gemm_tf32_kernel<1><<<grid, NTHREADS, smem, st>>>(maps, bias, rt, y, int(M), int(N), int(K), stages);
  }
  return check_launch(what);
}

}  // namespace tc
}  // namespace nes

using namespace nes;
using namespace nes::tc;

extern "C" int64_t nes_linear_fwd_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int mode) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int64_t a = align256(M * K * 4), b = align256(N * K * 4);
  return mode == 3 ? 2 * (a + b) : (a + b);
}

extern "C" int nes_linear_fwd_tc(const float* x, const float* weight, const float* bias, float* y,
                                 int64_t M, int64_t N, int64_t K, int mode,
                                 void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  NES_REQUIRE(M >= 0 && N >= 0 && K >= 0, NES_ERR_BAD_ARG, "linear_fwd_tc: negative extent");
  NES_REQUIRE(mode == 1 || mode == 3, NES_ERR_BAD_ARG, "linear_fwd_tc: mode must be 1 (TF32) or 3 (3xTF32)");
  if (M == 0 || N == 0) return NES_OK;
  NES_REQUIRE(x && weight && y, NES_ERR_BAD_ARG, "linear_fwd_tc: null pointer");
  NES_REQUIRE(K > 0 && K % 4 == 0, NES_ERR_UNSUPPORTED, "linear_fwd_tc: K=%lld must be a positive multiple of 4 (TMA row stride)", (long long)K);
  NES_REQUIRE(M <= INT32_MAX && N <= INT32_MAX && K <= INT32_MAX && ceil_div<int64_t>(N, BN) <= 65535, NES_ERR_UNSUPPORTED,
              "linear_fwd_tc: extent too large");
  const int64_t need = nes_linear_fwd_tc_scratch_bytes(M, N, K, mode);
  NES_REQUIRE(scratch && scratch_bytes >= need && (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, NES_ERR_SCRATCH,
              "linear_fwd_tc: scratch needs %lld bytes, 256-byte aligned", (long long)need);
  cudaStream_t st = as_stream(stream);
  // operand preparation: tf32-rounded copies (and residuals for the 3-term scheme)
  unsigned char* sp = static_cast<unsigned char*>(scratch);
  const int64_t a_bytes = align256(M * K * 4), b_bytes = align256(N * K * 4);
  float* a_hi = reinterpret_cast<float*>(sp);
  float* b_hi = reinterpret_cast<float*>(sp + a_bytes);
  float* a_lo = mode == 3 ? reinterpret_cast<float*>(sp + a_bytes + b_bytes) : nullptr;
  float* b_lo = mode == 3 ? reinterpret_cast<float*>(sp + 2 * a_bytes + b_bytes) : nullptr;
  split_tf32_kernel<<<(unsigned)ceil_div<int64_t>(M * K, 256), 256, 0, st>>>(x, a_hi, a_lo, M * K);
  int rc = check_launch("linear_fwd_tc(split x)");
  if (rc != NES_OK) return rc;
  split_tf32_kernel<<<(unsigned)ceil_div<int64_t>(N * K, 256), 256, 0, st>>>(weight, b_hi, b_lo, N * K);
  rc = check_launch("linear_fwd_tc(split w)");
  if (rc != NES_OK) return rc;

  const RowTerm none = {nullptr, 1, 1, 0};
  return run_gemm(a_hi, a_lo, b_hi, b_lo, bias, none, y, M, N, K, mode, st, "linear_fwd_tc");
}

extern "C" int nes_sparse_noise_add(float* y, const float* x, const int32_t* idx, const float* val, const float* bias_noise,
                                    int64_t D, int64_t R, int64_t in, int64_t out, int k, int antithetic, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0 && in >= 0 && out >= 0 && k >= 0, NES_ERR_BAD_ARG, "sparse_noise_add: negative extent");
  const int64_t total = D * R * out;
  if (total == 0) return NES_OK;
  NES_REQUIRE(y && x && (k == 0 || (idx && val)), NES_ERR_BAD_ARG, "sparse_noise_add: null pointer");
  NES_REQUIRE(ceil_div<int64_t>(total, 256) <= INT32_MAX, NES_ERR_UNSUPPORTED, "sparse_noise_add: too large");
  sparse_noise_add_kernel<<<(unsigned)ceil_div<int64_t>(total, 256), 256, 0, as_stream(stream)>>>(y, x, idx, val, bias_noise, D * R, D, R,
                                                                                                 in, out, k, antithetic);
  return check_launch("sparse_noise_add");
}

extern "C" int64_t nes_synthetic_linear_fwd_tc_scratch_bytes(int64_t D, int64_t R, int64_t in, int64_t out, int mode) {
  if (D <= 0 || R <= 0 || in <= 0 || out <= 0) return 0;
  const int64_t a = align256(D * R * in * 4), b = align256(out * in * 4), p = align256(D * R * out * 4);
  return (mode == 3 ? 2 : 1) * (a + b) + p;
}

// SyntheticLinear.forward on the tensor cores: y = x.W^T + bias, p = (x * fin).eps^T (two tcgen05 products on
// split operands), then y += s * (fout * p + beta).
extern "C" int nes_synthetic_linear_fwd_tc(const float* x, const float* weight, const float* bias, const float* eps,
                                           const float* bias_noise, const int8_t* fin, const int8_t* fout, float* y,
                                           int64_t D, int64_t R, int64_t in, int64_t out, int antithetic, int mode,
                                           void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0 && in >= 0 && out >= 0, NES_ERR_BAD_ARG, "synthetic_linear_fwd_tc: negative extent");
  NES_REQUIRE(mode == 1 || mode == 3, NES_ERR_BAD_ARG, "synthetic_linear_fwd_tc: mode must be 1 (TF32) or 3 (3xTF32)");
  if (D == 0 || R == 0 || out == 0) return NES_OK;
  NES_REQUIRE(x && weight && eps && y, NES_ERR_BAD_ARG, "synthetic_linear_fwd_tc: null pointer");
  NES_REQUIRE(in > 0 && in % 4 == 0, NES_ERR_UNSUPPORTED, "synthetic_linear_fwd_tc: in=%lld must be a positive multiple of 4", (long long)in);
  const int64_t B = D * R;
  NES_REQUIRE(B <= INT32_MAX && out <= INT32_MAX && in <= INT32_MAX && ceil_div<int64_t>(out, BN) <= 65535, NES_ERR_UNSUPPORTED,
              "synthetic_linear_fwd_tc: extent too large");
  const int64_t need = nes_synthetic_linear_fwd_tc_scratch_bytes(D, R, in, out, mode);
  NES_REQUIRE(scratch && scratch_bytes >= need && (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, NES_ERR_SCRATCH,
              "synthetic_linear_fwd_tc: scratch needs %lld bytes, 256-byte aligned", (long long)need);
  cudaStream_t st = as_stream(stream);
  unsigned char* sp = static_cast<unsigned char*>(scratch);
  const int64_t a_bytes = align256(B * in * 4), b_bytes = align256(out * in * 4);
  float* a_hi = reinterpret_cast<float*>(sp);
  float* b_hi = reinterpret_cast<float*>(sp + a_bytes);
  float* a_lo = mode == 3 ? reinterpret_cast<float*>(sp + a_bytes + b_bytes) : nullptr;
  float* b_lo = mode == 3 ? reinterpret_cast<float*>(sp + 2 * a_bytes + b_bytes) : nullptr;
  float* p = reinterpret_cast<float*>(sp + (mode == 3 ? 2 : 1) * (a_bytes + b_bytes));
  const unsigned ablocks = (unsigned)ceil_div<int64_t>(B * in, 256), bblocks = (unsigned)ceil_div<int64_t>(out * in, 256);
  const RowTerm none = {nullptr, 1, 1, 0};
  int rc;
  split_tf32_kernel<<<ablocks, 256, 0, st>>>(x, a_hi, a_lo, B * in);
  if ((rc = check_launch("synthetic_linear_fwd_tc(split x)")) != NES_OK) return rc;
  split_tf32_kernel<<<bblocks, 256, 0, st>>>(weight, b_hi, b_lo, out * in);
  if ((rc = check_launch("synthetic_linear_fwd_tc(split W)")) != NES_OK) return rc;
  if ((rc = run_gemm(a_hi, a_lo, b_hi, b_lo, bias, none, y, B, out, in, mode, st, "synthetic_linear_fwd_tc(base)")) != NES_OK) return rc;
  split_tf32_kernel<<<bblocks, 256, 0, st>>>(eps, b_hi, b_lo, out * in);
  if ((rc = check_launch("synthetic_linear_fwd_tc(split eps)")) != NES_OK) return rc;
  if (fin) {
    split_flipped_kernel<<<ablocks, 256, 0, st>>>(x, fin, a_hi, a_lo, B, D, in);
    if ((rc = check_launch("synthetic_linear_fwd_tc(flip x)")) != NES_OK) return rc;
  }
  if ((rc = run_gemm(a_hi, a_lo, b_hi, b_lo, nullptr, none, p, B, out, in, mode, st, "synthetic_linear_fwd_tc(noise)")) != NES_OK) return rc;
  synthetic_combine_kernel<<<(unsigned)ceil_div<int64_t>(B * out, 256), 256, 0, st>>>(y, p, fout, bias_noise, B, D, R, out, antithetic);
  return check_launch("synthetic_linear_fwd_tc(combine)");
}

// row length of the concatenated operand: a multiple of 16 bytes (4 fp32 / 8 bf16)
static int64_t permuted_k2(int64_t in, int64_t in_sp, int mode) {
  return (mode == 2 || mode == 4) ? ((in + in_sp + 7) & ~int64_t(7)) : ((in + in_sp + 3) & ~int64_t(3));
}

extern "C" int64_t nes_permuted_linear_fwd_tc_scratch_bytes(int64_t D, int64_t R, int64_t in, int64_t out, int64_t in_sp, int mode) {
  if (D <= 0 || R <= 0 || out <= 0 || in < 0 || in_sp < 0) return 0;
  const int64_t K2 = permuted_k2(in, in_sp, mode);
  const int64_t esz = (mode == 2 || mode == 4) ? 2 : 4;
  const int64_t a = align256(D * R * K2 * esz), b = align256(out * K2 * esz);
  return (mode == 3 || mode == 4) ? 2 * (a + b) : (a + b);
}

extern "C" int nes_permuted_linear_fwd_tc(const float* x, const float* weight, const float* bias, const float* eps,
                                          const float* bias_noise, const int16_t* pin, float* y,
                                          int64_t D, int64_t R, int64_t in, int64_t out, int64_t in_sp, int64_t out_sp,
                                          int antithetic, int mode, void* scratch, int64_t scratch_bytes,
                                          nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0 && in >= 0 && out >= 0 && in_sp >= 0 && out_sp >= 0 && out_sp <= out, NES_ERR_BAD_ARG,
              "permuted_linear_fwd_tc: bad extent");
  NES_REQUIRE(mode >= 1 && mode <= 4, NES_ERR_BAD_ARG,
              "permuted_linear_fwd_tc: mode must be 1 (TF32), 2 (bf16), 3 (3xTF32) or 4 (split-bf16, three products)");
  if (D == 0 || R == 0 || out == 0) return NES_OK;
  NES_REQUIRE(x && weight && eps && y, NES_ERR_BAD_ARG, "permuted_linear_fwd_tc: null pointer");
  NES_REQUIRE(pin || in_sp == in, NES_ERR_BAD_ARG, "permuted_linear_fwd_tc: in_sp != in without input permutations");
  NES_REQUIRE(in > 0 && in <= 32767 && in_sp <= INT32_MAX - in, NES_ERR_UNSUPPORTED, "permuted_linear_fwd_tc: in=%lld out of range", (long long)in);
  const int64_t B = D * R, K2 = permuted_k2(in, in_sp, mode);
  NES_REQUIRE(B <= INT32_MAX && out <= INT32_MAX && K2 <= INT32_MAX && ceil_div<int64_t>(out, BN) <= 65535, NES_ERR_UNSUPPORTED,
              "permuted_linear_fwd_tc: extent too large");
  const int64_t need = nes_permuted_linear_fwd_tc_scratch_bytes(D, R, in, out, in_sp, mode);
  NES_REQUIRE(scratch && scratch_bytes >= need && (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, NES_ERR_SCRATCH,
              "permuted_linear_fwd_tc: scratch needs %lld bytes, 256-byte aligned", (long long)need);
  cudaStream_t st = as_stream(stream);
  unsigned char* sp = static_cast<unsigned char*>(scratch);
  const bool half_words = (mode == 2 || mode == 4), split = (mode == 3 || mode == 4);
  const int64_t esz = half_words ? 2 : 4;
  const int64_t a_bytes = align256(B * K2 * esz), b_bytes = align256(out * K2 * esz);
  float* a_hi = reinterpret_cast<float*>(sp);
  float* b_hi = reinterpret_cast<float*>(sp + a_bytes);
  float* a_lo = split ? reinterpret_cast<float*>(sp + a_bytes + b_bytes) : nullptr;
  float* b_lo = split ? reinterpret_cast<float*>(sp + 2 * a_bytes + b_bytes) : nullptr;
  const unsigned blocks = (unsigned)(B < int64_t(sm_count()) * 16 ? B : int64_t(sm_count()) * 16);
  const unsigned fblocks = (unsigned)ceil_div<int64_t>(out * K2, 256);
  if (half_words) permuted_operand_kernel<true><<<blocks, 256, 0, st>>>(x, pin, a_hi, a_lo, B, D, R, int(in), int(in_sp), int(K2), antithetic);
  else permuted_operand_kernel<false><<<blocks, 256, 0, st>>>(x, pin, a_hi, a_lo, B, D, R, int(in), int(in_sp), int(K2), antithetic);
  int rc = check_launch("permuted_linear_fwd_tc(operand)");
  if (rc != NES_OK) return rc;
  if (half_words) permuted_filter_kernel<true><<<fblocks, 256, 0, st>>>(weight, eps, b_hi, b_lo, out, out_sp, int(in), int(in_sp), int(K2));
  else permuted_filter_kernel<false><<<fblocks, 256, 0, st>>>(weight, eps, b_hi, b_lo, out, out_sp, int(in), int(in_sp), int(K2));
  rc = check_launch("permuted_linear_fwd_tc(filter)");
  if (rc != NES_OK) return rc;
  const RowTerm rt = {bias_noise, D, R, antithetic};
  return run_gemm(a_hi, a_lo, b_hi, b_lo, bias, rt, y, B, out, K2, mode, st, "permuted_linear_fwd_tc");
}

namespace nes { namespace tc {
int conv_tc_error_word(int* v, bool clear);
int conv_bf16_error_word(int* v, bool clear);
int conv_pool_error_word(int* v, bool clear);
int permuted_out_error_word(int* v, bool clear);
} }

// Reads the error words of all tensor-core translation units, reports the first non-zero code and clears
// them, so that a later call reports only what has happened since this one.
extern "C" int nes_tc_error_flag(int* flag) {
  NES_REQUIRE(flag != nullptr, NES_ERR_BAD_ARG, "tc_error_flag: null pointer");
  int v[5] = {0, 0, 0, 0, 0};
  int rc = read_error_word(&v[0], true, "tc_error_flag");
  if (rc != NES_OK) return rc;
  if ((rc = nes::tc::conv_tc_error_word(&v[1], true)) != NES_OK) return rc;
  if ((rc = nes::tc::conv_bf16_error_word(&v[2], true)) != NES_OK) return rc;
  if ((rc = nes::tc::conv_pool_error_word(&v[3], true)) != NES_OK) return rc;
  if ((rc = nes::tc::permuted_out_error_word(&v[4], true)) != NES_OK) return rc;
  *flag = 0;
  for (int i = 0; i < 5; ++i)
    if (v[i]) { *flag = v[i]; break; }
  return NES_OK;
}
