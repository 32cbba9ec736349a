// Tensor-core GEMM for sm_100a: C[M,N] = A[M,K] . B[N,K]^T (+ bias), fp32 in / fp32 out.
//
// Blackwell execution model, written directly in PTX:
//   * operands travel global -> shared memory as 128-byte-swizzled tiles by TMA
//     (cp.async.bulk.tensor.2d, one elected producer thread, mbarrier transaction counts);
//   * one elected thread issues tcgen05.mma (kind::tf32, M = 128, N = 128, K = 8 per
//     instruction) with both operands read from shared memory through matrix descriptors and
//     the fp32 accumulator tile (128 lanes x 128 columns) living in tensor memory;
//   * tcgen05.commit hands shared-memory stages back to the producer and signals the epilogue;
//   * four epilogue warps read the accumulator with tcgen05.ld (one TMEM lane = one output
//     row per thread), add the bias and store.
// Precision modes: TERMS = 1 is plain TF32 (inputs rounded to 10 mantissa bits; relative error
// ~1e-3, for callers that state it).  TERMS = 3 is the error-compensated 3xTF32 scheme: every
// operand is split beforehand into hi = tf32(a) and lo = a - hi, and the kernel accumulates
// a_lo.b_hi + a_hi.b_lo + a_hi.b_hi, which keeps fp32-level accuracy (~1e-6) on the tensor pipe.
//
// Every wait on an mbarrier is bounded: when the limit is hit the thread records an error code
// in a device word (read by nes_tc_error_flag), stops issuing work and falls through to the
// common exit, where tensor memory is released.
#include <cuda.h>
#include "common.cuh"

namespace nes {
namespace tc {

constexpr int BM = 128, BN = 128, BKE = 32;          // tile, K elements (fp32) per stage = one 128-byte swizzle row
constexpr int TILE_BYTES = BM * BKE * 4;             // 16 KiB per operand tile
constexpr int NTHREADS = 192;                        // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;   // about one second at B200 clocks

__device__ int g_tc_error = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false = gave up (error recorded).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int code) {
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > WAIT_LIMIT_CYCLES) break;
  }
  atomicCAS(&g_tc_error, 0, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are one 128-byte swizzle span:
// start address (>>4), leading byte offset 16 B (unused for this layout), stride byte offset
// 1024 B between 8-row groups, descriptor version 1, layout type 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= uint64_t((saddr & 0x3FFFFu) >> 4);
  d |= uint64_t(1) << 16;
  d |= uint64_t(1024 >> 4) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

// Instruction descriptor: D = fp32, A = B = tf32, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t idesc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

struct Maps { CUtensorMap a_hi, b_hi, a_lo, b_lo; };

template <int TERMS>
__global__ void __launch_bounds__(NTHREADS, 1) gemm_tf32_kernel(const __grid_constant__ Maps maps, const float* __restrict__ bias,
                                                                 float* __restrict__ C, int M, int N, int K, int stages) {
  extern __shared__ unsigned char dyn_raw[];
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
  const int nk = (K + BKE - 1) / BKE;

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
        tma_load_2d(st, &maps.a_hi, &full[s], kt * BKE, m0);
        tma_load_2d(st + TILE_BYTES, &maps.b_hi, &full[s], kt * BKE, n0);
        if (TERMS == 3) {
          tma_load_2d(st + 2 * TILE_BYTES, &maps.a_lo, &full[s], kt * BKE, m0);
          tma_load_2d(st + 3 * TILE_BYTES, &maps.b_lo, &full[s], kt * BKE, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc = idesc_tf32(BM, BN);
      bool ok = true;
      for (int kt = 0; kt < nk && ok; ++kt) {
        const int s = kt % stages;
        const uint32_t ph = (kt / stages) & 1;
        ok = mbar_wait(&full[s], ph, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t st = smem_u32(tiles + size_t(s) * STAGE_BYTES);
        const uint64_t a_hi = smem_desc_sw128(st), b_hi = smem_desc_sw128(st + TILE_BYTES);
#pragma unroll
        for (int k = 0; k < BKE / 8; ++k) {            // advance 32 bytes (2 descriptor units) per K = 8
          const uint64_t adv = uint64_t(k * 2);
          if (TERMS == 3) {
            const uint64_t a_lo = smem_desc_sw128(st + 2 * TILE_BYTES), b_lo = smem_desc_sw128(st + 3 * TILE_BYTES);
            mma_tf32(tmem_base, a_lo + adv, b_hi + adv, idesc, (kt > 0 || k > 0) ? 1u : 0u);
            mma_tf32(tmem_base, a_hi + adv, b_lo + adv, idesc, 1u);
            mma_tf32(tmem_base, a_hi + adv, b_hi + adv, idesc, 1u);
          } else {
            mma_tf32(tmem_base, a_hi + adv, b_hi + adv, idesc, (kt > 0 || k > 0) ? 1u : 0u);
          }
        }
        mma_commit(&empty[s]);            // frees the stage once these MMAs have read it
      }
      mma_commit(accum);                  // accumulator complete (or abandoned: epilogue checks the error word)
    }
  } else {
    // ---- epilogue: warp w may touch TMEM lanes 32*(w%4) .. +31
    const int q = warp & 3;
    const bool ok = mbar_wait(accum, 0, 3);
    tc_fence_after();
    if (ok && g_tc_error == 0 && nk > 0) {
      const int64_t gm = int64_t(m0) + q * 32 + lane;
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
        for (int j = 0; j < BN; ++j) if (n0 + j < N) C[gm * N + n0 + j] = bias ? bias[n0 + j] : 0.f;
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
  uint32_t u = __float_as_uint(a);
  if ((u & 0x7F800000u) != 0x7F800000u) u = (u + 0x0FFFu + ((u >> 13) & 1u)) & 0xFFFFE000u;
  const float h = __uint_as_float(u);
  hi[i] = h;
  if (lo) lo[i] = a - h;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D fp32 row-major [rows][cols] tensor, box = 32 columns x box_rows rows, 128-byte swizzle, zero fill
static int make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int box_rows, const char* what) {
  EncodeTiledFn fn = encode_fn();
  NES_REQUIRE(fn != nullptr, NES_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", what);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)BKE, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NES_REQUIRE(r == CUDA_SUCCESS, NES_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
  return NES_OK;
}

static int64_t align256(int64_t v) { return (v + 255) & ~int64_t(255); }

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

  Maps maps;
  if ((rc = make_map(&maps.a_hi, a_hi, M, K, BM, "linear_fwd_tc")) != NES_OK) return rc;
  if ((rc = make_map(&maps.b_hi, b_hi, N, K, BN, "linear_fwd_tc")) != NES_OK) return rc;
  if (mode == 3) {
    if ((rc = make_map(&maps.a_lo, a_lo, M, K, BM, "linear_fwd_tc")) != NES_OK) return rc;
    if ((rc = make_map(&maps.b_lo, b_lo, N, K, BN, "linear_fwd_tc")) != NES_OK) return rc;
  } else {
    maps.a_lo = maps.a_hi;
    maps.b_lo = maps.b_hi;
  }
  const int stages = (mode == 3) ? 3 : 4;
  const int stage_bytes = (mode == 3 ? 4 : 2) * TILE_BYTES;
  const size_t smem = 1024 + size_t(stages) * stage_bytes + (2 * stages + 1) * sizeof(uint64_t) + 16;
  dim3 grid((unsigned)ceil_div<int64_t>(M, BM), (unsigned)ceil_div<int64_t>(N, BN));
  cudaError_t e;
  if (mode == 3) {
    e = cudaFuncSetAttribute(gemm_tf32_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "linear_fwd_tc: shared memory opt-in failed: %s", cudaGetErrorString(e));
    gemm_tf32_kernel<3><<<grid, NTHREADS, smem, st>>>(maps, bias, y, int(M), int(N), int(K), stages);
  } else {
    e = cudaFuncSetAttribute(gemm_tf32_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "linear_fwd_tc: shared memory opt-in failed: %s", cudaGetErrorString(e));
    gemm_tf32_kernel<1><<<grid, NTHREADS, smem, st>>>(maps, bias, y, int(M), int(N), int(K), stages);
  }
  return check_launch("linear_fwd_tc");
}

extern "C" int nes_tc_error_flag(int* flag) {
  NES_REQUIRE(flag != nullptr, NES_ERR_BAD_ARG, "tc_error_flag: null pointer");
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int));
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "tc_error_flag: %s", cudaGetErrorString(e));
  *flag = v;
  return NES_OK;
}
