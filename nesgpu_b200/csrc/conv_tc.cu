// Tensor-core convolution for the per-member layers (PermutedConv2d / PerturbedConv2d), TF32 mode.
//
// The population forward is, per member d and antithetic sign s, an ordinary convolution with the
// member's effective filter W_d = W + s * E_d.  A persistent thread block takes (member, sign) units:
//   1. its four "builder" warps form W_d in shared memory -- from W and the shared noise through the
//      member's channel maps, or from the member's dense noise -- already rounded to TF32, reordered to
//      k = tap * Cin + c and laid out as the 128-byte-swizzled K-major tiles tcgen05.mma reads
//      (never materialised in HBM);
//   2. a producer thread streams the member's input as im2col tiles straight out of a channels-last
//      copy of x: one 4-D TMA box {32 channels, BW, BH, 1 image} per (tile, tap, channel chunk),
//      shifted by the tap, with the zero padding supplied by TMA's out-of-bounds fill;
//   3. one thread issues tcgen05.mma (kind::tf32, M = 128 pixels, N = Cout, K = 8) into one of two
//      accumulator tiles in tensor memory, so that
//   4. the builder warps, now epilogue warps, read the other accumulator with tcgen05.ld (one pixel per
//      thread), add bias + s * bias_noise and store NCHW rows while the next tile is multiplied.
// A pre-pass writes the channels-last, TF32-rounded copy of x (the only extra HBM traffic).
// All mbarrier waits are bounded (see tc_ptx.cuh); an error code is left in the device error word.
#include "tc_ptx.cuh"

namespace nes {

// defined in conv.cu
int launch_permuted_maps(const int16_t* pin, const int16_t* pout, int16_t* omap, int16_t* imap, int64_t D,
                         int Cin, int Cout, int in_sp, int out_sp, cudaStream_t st);

namespace tc {

constexpr int CONV_THREADS = 192;
constexpr int A_TILE_BYTES = 128 * 128;   // 128 pixels x 32 fp32 channels

struct ConvTcParams {
  int Cin, H, W, Cout, kh, kw, ph, pw, dh, dw, Ho, Wo;
  int BW, BH, tiles_w, tiles_h;
  long long D, R;
  int antithetic, sign_groups, units;
  int stages, kchunks, cchunks, tmem_cols;
  const float* weight; const float* bias; const float* bias_noise; float* y;
  int noise_kind;               // 0 none, 1 dense (D,Cout,Cin,ksz), 2 permuted (out_sp,in_sp,ksz) through omap / imap
  const float* noise; const int16_t* omap; const int16_t* imap; int in_sp;
};

// repeats [r0, r1) that belong to sign group sg, and the sign
__device__ __forceinline__ void unit_range(const ConvTcParams& p, int sg, long long& r0, long long& r1, float& s) {
  if (!p.antithetic) { r0 = 0; r1 = p.R; s = 1.f; return; }
  const long long half = (p.R + 1) / 2;
  if (sg == 0) { r0 = 0; r1 = half; s = 1.f; } else { r0 = half; r1 = p.R; s = -1.f; }
}

__global__ void __launch_bounds__(CONV_THREADS, 1) conv_tf32_kernel(const __grid_constant__ CUtensorMap xmap, const ConvTcParams p) {
  extern __shared__ unsigned char dyn_raw[];
  const uint32_t raw = smem_u32(dyn_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  unsigned char* wd = dyn_raw + pad;                                   // [kchunks][Cout][128 B]
  const int wd_chunk_bytes = p.Cout * 128;
  unsigned char* atiles = wd + size_t(p.kchunks) * wd_chunk_bytes;     // [stages][16 KiB]
  uint64_t* full = reinterpret_cast<uint64_t*>(atiles + size_t(p.stages) * A_TILE_BYTES);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;     // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint64_t* wd_ready = acc_empty + 2;
  uint64_t* wd_free = wd_ready + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(wd_free + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ksz = p.kh * p.kw;
  const int K = p.Cin * ksz;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    mbar_init(wd_ready, 4);
    mbar_init(wd_free, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, (uint32_t)p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      uint32_t g = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        const long long d = u / p.sign_groups;
        long long r0, r1; float s;
        unit_range(p, u % p.sign_groups, r0, r1, s);
        for (long long r = r0; r < r1 && ok; ++r) {
          const int b = int(r * p.D + d);
          for (int th = 0; th < p.tiles_h && ok; ++th)
            for (int tw = 0; tw < p.tiles_w && ok; ++tw)
              for (int tap = 0; tap < ksz && ok; ++tap) {
                const int i = tap / p.kw, j = tap - i * p.kw;
                const int x0 = tw * p.BW + j * p.dw - p.pw;
                const int y0 = th * p.BH + i * p.dh - p.ph;
                for (int cc = 0; cc < p.cchunks; ++cc, ++g) {
                  const int st = g % p.stages;
                  const uint32_t phs = (g / p.stages) & 1;
                  if (!mbar_wait(&empty[st], phs ^ 1, 1)) { ok = false; break; }
                  mbar_expect_tx(&full[st], A_TILE_BYTES);
                  tma_load_4d(atiles + size_t(st) * A_TILE_BYTES, &xmap, &full[st], cc * 32, x0, y0, b);
                }
              }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(p.Cout >> 3) << 17) | (uint32_t(128 >> 4) << 24);
      uint32_t g = 0, t = 0, ul = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        long long r0, r1; float s;
        unit_range(p, u % p.sign_groups, r0, r1, s);
        if (r1 <= r0) continue;
        if (!mbar_wait(wd_ready, ul & 1, 2)) { ok = false; break; }
        tc_fence_after();
        const long long ntiles = (r1 - r0) * p.tiles_h * p.tiles_w;
        for (long long ti = 0; ti < ntiles && ok; ++ti, ++t) {
          const uint32_t buf = t & 1;
          if (!mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, 2)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + buf * uint32_t(p.Cout);
          for (int jc = 0; jc < p.kchunks; ++jc, ++g) {
            const int st = g % p.stages;
            const uint32_t phs = (g / p.stages) & 1;
            if (!mbar_wait(&full[st], phs, 2)) { ok = false; break; }
            tc_fence_after();
            const uint64_t adesc = smem_desc_sw128(smem_u32(atiles + size_t(st) * A_TILE_BYTES));
            const uint64_t bdesc = smem_desc_sw128(smem_u32(wd + size_t(jc) * wd_chunk_bytes));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_tf32(tmem_d, adesc + uint64_t(2 * k), bdesc + uint64_t(2 * k), idesc, (jc > 0 || k > 0) ? 1u : 0u);
            mma_commit(&empty[st]);
          }
          mma_commit(&acc_full[buf]);
        }
        mma_commit(wd_free);
        ++ul;
      }
    }
  } else {
    // ---------------------------------------------------------------------- filter builders / epilogue
    const int te = threadIdx.x - 64;            // 0..127
    const int q = warp & 3;                     // TMEM lane quadrant this warp may read
    const int pix = q * 32 + lane;              // pixel of the tile = accumulator row
    const int ty = pix / p.BW, tx = pix - ty * p.BW;
    uint32_t t = 0, ul = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      const long long d = u / p.sign_groups;
      long long r0, r1; float s;
      unit_range(p, u % p.sign_groups, r0, r1, s);
      if (r1 <= r0) continue;
      if (!mbar_wait(wd_free, (ul & 1) ^ 1, 4)) { ok = false; break; }
      // W_d[n][tap*Cin + c] = tf32(W[n][c][tap] + s * noise_d[n][c][tap])
      const int total = p.Cout * K;
      for (int idx = te; idx < total; idx += 128) {
        const int n = idx / K;
        const int rem = idx - n * K;
        const int c = rem / ksz, tap = rem - c * ksz;
        float v = __ldg(p.weight + idx);
        if (p.noise_kind == 1) {
          v += s * __ldg(p.noise + size_t(d) * total + idx);
        } else if (p.noise_kind == 2) {
          const int so = p.omap[d * p.Cout + n];
          const int ci = p.imap[d * p.Cin + c];
          if (so >= 0 && ci >= 0) v += s * __ldg(p.noise + (size_t(so) * p.in_sp + ci) * ksz + tap);
        }
        const int kk = tap * p.Cin + c;
        const int jc = kk >> 5, w32 = kk & 31;
        unsigned char* dst = wd + size_t(jc) * wd_chunk_bytes + (n >> 3) * 1024 + (n & 7) * 128 +
                             ((((w32 >> 2) ^ (n & 7))) << 4) + (w32 & 3) * 4;
        *reinterpret_cast<float*>(dst) = round_tf32(v);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(wd_ready);

      for (long long r = r0; r < r1 && ok; ++r) {
        const long long b = r * p.D + d;
        for (int th = 0; th < p.tiles_h && ok; ++th)
          for (int tw = 0; tw < p.tiles_w && ok; ++tw, ++t) {
            const uint32_t buf = t & 1;
            if (!mbar_wait(&acc_full[buf], (t >> 1) & 1, 3)) { ok = false; break; }
            tc_fence_after();
            const int oy = th * p.BH + ty, ox = tw * p.BW + tx;
            const bool valid = (oy < p.Ho) && (ox < p.Wo) && (g_tc_error == 0);
            for (int c0 = 0; c0 < p.Cout; c0 += 32) {
              uint32_t acc[32];
              tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + buf * uint32_t(p.Cout) + uint32_t(c0), acc);
              if (valid) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const int n = c0 + j;
                  float v = __uint_as_float(acc[j]);
                  if (p.bias) v += __ldg(p.bias + n);
                  if (p.bias_noise) v += s * __ldg(p.bias_noise + d * p.Cout + n);
                  p.y[((size_t(b) * p.Cout + n) * p.Ho + oy) * p.Wo + ox] = v;
                }
              }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
          }
      }
      ++ul;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// x (B,C,H,W) -> channels-last (B,H,W,C), rounded to TF32.  32x32 tiles through shared memory so that both
// the reads (along HW) and the writes (along C) are coalesced.
__global__ void nchw_to_nhwc_tf32_kernel(const float* __restrict__ x, float* __restrict__ out, int C, int HW) {
  __shared__ float tile[32][33];
  const size_t b = blockIdx.z;
  const int hw0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const float* src = x + b * size_t(C) * HW;
  float* dst = out + b * size_t(C) * HW;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, hw = hw0 + threadIdx.x;
    tile[i][threadIdx.x] = (c < C && hw < HW) ? src[size_t(c) * HW + hw] : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int hw = hw0 + i, c = c0 + threadIdx.x;
    if (hw < HW && c < C) dst[size_t(hw) * C + c] = round_tf32(tile[threadIdx.x][i]);
  }
}

int conv_tc_error_word(int* v) {
  cudaError_t e = cudaMemcpyFromSymbol(v, g_tc_error, sizeof(int));
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "tc_error_flag: %s", cudaGetErrorString(e));
  return NES_OK;
}

static int64_t align256(int64_t v) { return (v + 255) & ~int64_t(255); }

struct ConvTcPlan { ConvTcParams p; size_t smem; int64_t x_bytes, map_bytes; };

static int plan_conv_tc(ConvTcPlan& pl, int64_t D, int64_t R, int Cin, int H, int W, int Cout, int kh, int kw,
                        int sh, int sw, int ph, int pw, int dh, int dw, int antithetic, const char* what) {
  NES_REQUIRE(D >= 0 && R >= 0 && Cin > 0 && H > 0 && W > 0 && Cout > 0 && kh > 0 && kw > 0 && ph >= 0 && pw >= 0 &&
              dh > 0 && dw > 0, NES_ERR_BAD_ARG, "%s: bad geometry", what);
  NES_REQUIRE(sh == 1 && sw == 1, NES_ERR_UNSUPPORTED, "%s: the tensor-core path needs stride 1", what);
  NES_REQUIRE(Cin % 32 == 0, NES_ERR_UNSUPPORTED, "%s: the tensor-core path needs Cin %% 32 == 0 (got %d)", what, Cin);
  NES_REQUIRE(Cout % 32 == 0 && Cout <= 256, NES_ERR_UNSUPPORTED, "%s: the tensor-core path needs Cout %% 32 == 0 and <= 256 (got %d)", what, Cout);
  ConvTcParams& p = pl.p;
  p.Cin = Cin; p.H = H; p.W = W; p.Cout = Cout; p.kh = kh; p.kw = kw; p.ph = ph; p.pw = pw; p.dh = dh; p.dw = dw;
  p.Ho = H + 2 * ph - dh * (kh - 1);
  p.Wo = W + 2 * pw - dw * (kw - 1);
  NES_REQUIRE(p.Ho > 0 && p.Wo > 0, NES_ERR_BAD_ARG, "%s: empty output", what);
  int bw = 8;
  while (bw < p.Wo && bw < 128) bw <<= 1;
  p.BW = bw; p.BH = 128 / bw;
  p.tiles_w = ceil_div(p.Wo, p.BW); p.tiles_h = ceil_div(p.Ho, p.BH);
  p.D = D; p.R = R; p.antithetic = antithetic;
  p.sign_groups = antithetic ? 2 : 1;
  NES_REQUIRE(D * p.sign_groups <= INT32_MAX && D * R <= INT32_MAX, NES_ERR_UNSUPPORTED, "%s: population too large", what);
  p.units = int(D * p.sign_groups);
  p.cchunks = Cin / 32;
  p.kchunks = kh * kw * p.cchunks;
  int cols = 32;
  while (cols < 2 * Cout) cols <<= 1;
  p.tmem_cols = cols;
  const size_t wd_bytes = size_t(p.kchunks) * Cout * 128;
  const size_t fixed = 1024 + wd_bytes + 64 /* barriers */ + 16;
  const size_t limit = 227 * 1024;
  NES_REQUIRE(fixed + 2 * (A_TILE_BYTES + 16) <= limit, NES_ERR_UNSUPPORTED,
              "%s: the member filter (%zu bytes) does not fit in shared memory on the tensor-core path", what, wd_bytes);
  int stages = int((limit - fixed) / (A_TILE_BYTES + 16));
  if (stages > 8) stages = 8;
  p.stages = stages;
  pl.smem = 1024 + wd_bytes + size_t(stages) * A_TILE_BYTES + (2 * stages + 6) * sizeof(uint64_t) + 16;
  pl.x_bytes = align256(D * R * int64_t(Cin) * H * W * 4);
  pl.map_bytes = align256(D * (int64_t(Cin) + Cout) * 2);
  return NES_OK;
}

static int run_conv_tc(ConvTcPlan& pl, const float* x, float* x_nhwc, cudaStream_t st, const char* what) {
  ConvTcParams& p = pl.p;
  const int64_t B = p.D * p.R;
  const int HW = p.H * p.W;
  NES_REQUIRE(B <= 65535, NES_ERR_UNSUPPORTED, "%s: more than 65535 images per call on the tensor-core path", what);
  dim3 tgrid((unsigned)ceil_div(HW, 32), (unsigned)ceil_div(p.Cin, 32), (unsigned)B);
  nchw_to_nhwc_tf32_kernel<<<tgrid, dim3(32, 8), 0, st>>>(x, x_nhwc, p.Cin, HW);
  int rc = check_launch(what);
  if (rc != NES_OK) return rc;

  EncodeTiledFn fn = encode_fn();
  NES_REQUIRE(fn != nullptr, NES_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", what);
  CUtensorMap xmap;
  cuuint64_t dims[4] = {(cuuint64_t)p.Cin, (cuuint64_t)p.W, (cuuint64_t)p.H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)p.Cin * 4, (cuuint64_t)p.W * p.Cin * 4, (cuuint64_t)p.H * p.W * p.Cin * 4};
  cuuint32_t box[4] = {32, (cuuint32_t)p.BW, (cuuint32_t)p.BH, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, x_nhwc, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NES_REQUIRE(r == CUDA_SUCCESS, NES_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);

  cudaError_t e = cudaFuncSetAttribute(conv_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "%s: shared memory opt-in failed: %s", what, cudaGetErrorString(e));
  int grid = p.units < sm_count() ? p.units : sm_count();
  if (grid < 1) grid = 1;
  conv_tf32_kernel<<<grid, CONV_THREADS, pl.smem, st>>>(xmap, p);
  return check_launch(what);
}

}  // namespace tc
}  // namespace nes

using namespace nes;
using namespace nes::tc;

extern "C" int64_t nes_conv2d_fwd_tc_scratch_bytes(int64_t D, int64_t R, int Cin, int H, int W, int Cout) {
  if (D <= 0 || R <= 0) return 0;
  return align256(D * R * int64_t(Cin) * H * W * 4) + align256(D * (int64_t(Cin) + Cout) * 2);
}

extern "C" int nes_perturbed_conv2d_fwd_tc(const float* x, const float* weight, const float* bias,
                                           const float* noise, const float* bias_noise, float* y,
                                           int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                           int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                           int antithetic, void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  ConvTcPlan pl;
  int rc = plan_conv_tc(pl, D, R, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, antithetic, "perturbed_conv2d_fwd_tc");
  if (rc != NES_OK) return rc;
  if (D == 0 || R == 0) return NES_OK;
  NES_REQUIRE(x && weight && noise && y, NES_ERR_BAD_ARG, "perturbed_conv2d_fwd_tc: null pointer");
  NES_REQUIRE(scratch && scratch_bytes >= pl.x_bytes && (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, NES_ERR_SCRATCH,
              "perturbed_conv2d_fwd_tc: scratch needs %lld bytes, 256-byte aligned", (long long)pl.x_bytes);
  pl.p.weight = weight; pl.p.bias = bias; pl.p.bias_noise = bias_noise; pl.p.y = y;
  pl.p.noise_kind = 1; pl.p.noise = noise; pl.p.omap = nullptr; pl.p.imap = nullptr; pl.p.in_sp = Cin;
  return run_conv_tc(pl, x, static_cast<float*>(scratch), as_stream(stream), "perturbed_conv2d_fwd_tc");
}

extern "C" int nes_permuted_conv2d_fwd_tc(const float* x, const float* weight, const float* bias,
                                          const float* eps, const float* bias_noise,
                                          const int16_t* pin, const int16_t* pout, float* y,
                                          int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                          int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                          int in_sp, int out_sp, int antithetic,
                                          void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  ConvTcPlan pl;
  int rc = plan_conv_tc(pl, D, R, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, antithetic, "permuted_conv2d_fwd_tc");
  if (rc != NES_OK) return rc;
  if (D == 0 || R == 0) return NES_OK;
  NES_REQUIRE(x && weight && eps && y, NES_ERR_BAD_ARG, "permuted_conv2d_fwd_tc: null pointer");
  NES_REQUIRE(out_sp >= 0 && out_sp <= Cout && in_sp >= 0 && in_sp <= Cin && (pin || in_sp == Cin), NES_ERR_BAD_ARG,
              "permuted_conv2d_fwd_tc: sparsity exceeds degree");
  NES_REQUIRE(scratch && scratch_bytes >= pl.x_bytes + pl.map_bytes && (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0,
              NES_ERR_SCRATCH, "permuted_conv2d_fwd_tc: scratch needs %lld bytes, 256-byte aligned",
              (long long)(pl.x_bytes + pl.map_bytes));
  cudaStream_t st = as_stream(stream);
  int16_t* omap = reinterpret_cast<int16_t*>(static_cast<unsigned char*>(scratch) + pl.x_bytes);
  int16_t* imap = omap + D * Cout;
  rc = launch_permuted_maps(pin, pout, omap, imap, D, Cin, Cout, in_sp, out_sp, st);
  if (rc != NES_OK) return rc;
  pl.p.weight = weight; pl.p.bias = bias; pl.p.bias_noise = bias_noise; pl.p.y = y;
  pl.p.noise_kind = 2; pl.p.noise = eps; pl.p.omap = omap; pl.p.imap = imap; pl.p.in_sp = in_sp;
  return run_conv_tc(pl, x, static_cast<float*>(scratch), st, "permuted_conv2d_fwd_tc");
}
