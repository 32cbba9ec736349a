// Out-permuted convolution of an input that every member shares, fused with ReLU and 2x2 max-pooling.
//
// With output permutations only, member d's convolution of a shared image is
//   conv(x, W)[c] + s * conv(x, eps)[pout[d, c]] + bias[c] + s * bias_noise[d, c],
// so the two convolutions are computed once per image (one plain convolution with the stacked filter
// [W; eps]) and the per-member work is a gather, an add, the ReLU and the pooling.  A block keeps the
// stacked feature maps of one image in shared memory and walks a group of members; lanes are channels, so
// every store is a run of consecutive channels of one pooled pixel: the output is channels-last.  With an
// even row length the rows of a pooling window are read as 8-byte pairs.
#include <cuda_bf16.h>
#include "common.cuh"

namespace nes {

__device__ inline float round_to_tf32(float a) {
  uint32_t u = __float_as_uint(a);
  u += 0x00000FFFu + ((u >> 13) & 1u);
  return __uint_as_float(u & 0xFFFFE000u);
}

// even pitch >= hw with pitch / 2 odd: planes start 8-byte aligned and the 16 lanes of a 64-bit
// shared-memory phase (16 channels) fall on 16 different bank pairs
__host__ __device__ inline int plane_pitch(int hw) {
  int p = (hw + 1) & ~1;
  if (((p >> 1) & 1) == 0) p += 2;
  return p;
}

// MODE: 0 = fp32, 1 = fp32 rounded to TF32, 2 = bf16
template <int MODE> struct OutType { typedef float type; };
template <> struct OutType<2> { typedef __nv_bfloat16 type; };

template <int MODE>
__device__ __forceinline__ typename OutType<MODE>::type pool_value(float a0, float a1, float a2, float a3, float add) {
  const float v = fmaxf(fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)) + add, 0.f);
  if constexpr (MODE == 2) return __float2bfloat16_rn(v);
  else if constexpr (MODE == 1) return round_to_tf32(v);
  else return v;
}

constexpr int CP_WARPS = 32;          // warps per block

template <int MODE>
__global__ void __launch_bounds__(CP_WARPS * 32) shared_conv_pool_kernel(
    const float* __restrict__ z, const float* __restrict__ bias, const float* __restrict__ bias_noise,
    const int16_t* __restrict__ pout, typename OutType<MODE>::type* __restrict__ y, int64_t R, int64_t D, int Cout, int osp,
    int Ho, int Wo, int antithetic, int members_per_block) {
  typedef typename OutType<MODE>::type out_t;
  extern __shared__ __align__(16) float planes[];                 // (Cout + osp) planes of Ho*Wo (+1 pad) floats
  const int hw = Ho * Wo, pitch = plane_pitch(hw);
  const int Hp = Ho / 2, Wp = Wo / 2, pooled = Hp * Wp;
  const int64_t r = blockIdx.x;
  const float* zr = z + r * int64_t(Cout + osp) * hw;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int c = warp; c < Cout + osp; c += warps)
    for (int p = lane; p < hw; p += 32) planes[c * pitch + p] = zr[c * hw + p];
  __syncthreads();
  const float sgn = anti_sign(r, R, antithetic);
  const int64_t d0 = int64_t(blockIdx.y) * members_per_block;
  const int64_t d1 = (d0 + members_per_block < D) ? d0 + members_per_block : D;
  // a warp owns whole members, so the latency of a member's permutation / bias loads is hidden by the
  // other warps' arithmetic
  for (int64_t d = d0 + warp; d < d1; d += warps) {
    for (int c0 = 0; c0 < Cout; c0 += 32) {
      const int c = c0 + lane;
      const bool live = c < Cout;
      const float* base = planes + (live ? c : 0) * pitch;
      int so = live ? (pout ? int(pout[d * Cout + c]) : c) : 0;
      const bool noisy = live && so < osp;
      const float* noise = planes + (Cout + (noisy ? so : 0)) * pitch;
      const float s = noisy ? sgn : 0.f;
      float add = (live && bias) ? bias[c] : 0.f;
      if (live && bias_noise) add += sgn * bias_noise[d * Cout + c];
      out_t* out = y + ((r * D + d) * pooled) * Cout + c;
      if ((Wo & 1) == 0) {
        // even row length: both rows of a window start on 8-byte boundaries
        for (int py = 0; py < Hp; ++py) {
          const float* b = base + (2 * py) * Wo;
          const float* n = noise + (2 * py) * Wo;
          out_t* o = out + int64_t(py) * Wp * Cout;
#pragma unroll 4
          for (int px = 0; px < Wp; ++px, b += 2, n += 2, o += Cout) {
            const float2 b0 = *reinterpret_cast<const float2*>(b);
            const float2 b1 = *reinterpret_cast<const float2*>(b + Wo);
            const float2 n0 = *reinterpret_cast<const float2*>(n);
            const float2 n1 = *reinterpret_cast<const float2*>(n + Wo);
            const out_t v = pool_value<MODE>(fmaf(s, n0.x, b0.x), fmaf(s, n0.y, b0.y), fmaf(s, n1.x, b1.x), fmaf(s, n1.y, b1.y), add);
            if (live) o[0] = v;
          }
        }
        continue;
      }
      for (int py = 0; py < Hp; ++py) {
        const int row = (2 * py) * Wo;
#pragma unroll 4
        for (int px = 0; px < Wp; ++px) {
          const int p00 = row + 2 * px;
          const float v0 = base[p00] + s * noise[p00];
          const float v1 = base[p00 + 1] + s * noise[p00 + 1];
          const float v2 = base[p00 + Wo] + s * noise[p00 + Wo];
          const float v3 = base[p00 + Wo + 1] + s * noise[p00 + Wo + 1];
          const out_t v = pool_value<MODE>(v0, v1, v2, v3, add);
          if (live) out[int64_t(py * Wp + px) * Cout] = v;
        }
      }
    }
  }
}

}  // namespace nes

using namespace nes;

extern "C" int nes_shared_conv_pool_fwd(const float* z, const float* bias, const float* bias_noise,
                                        const int16_t* pout, void* y, int64_t R, int64_t D, int Cout, int out_sp,
                                        int Ho, int Wo, int antithetic, int out_mode, nes_stream_t stream) {
  NES_REQUIRE(R >= 0 && D >= 0 && Cout >= 0 && out_sp >= 0 && Ho >= 0 && Wo >= 0, NES_ERR_BAD_ARG,
              "shared_conv_pool_fwd: negative extent");
  NES_REQUIRE(out_sp <= Cout, NES_ERR_BAD_ARG, "shared_conv_pool_fwd: out_sp exceeds the channel count");
  NES_REQUIRE(out_mode >= 0 && out_mode <= 2, NES_ERR_BAD_ARG, "shared_conv_pool_fwd: out_mode must be 0 (fp32), 1 (tf32) or 2 (bf16)");
  if (R == 0 || D == 0 || Cout == 0 || Ho < 2 || Wo < 2) return NES_OK;
  NES_REQUIRE(z && y, NES_ERR_BAD_ARG, "shared_conv_pool_fwd: null pointer");
  NES_REQUIRE(R <= INT32_MAX, NES_ERR_UNSUPPORTED, "shared_conv_pool_fwd: too many images");
  const int64_t hw = int64_t(Ho) * Wo;
  const size_t smem = size_t(Cout + out_sp) * size_t(plane_pitch(int(hw))) * sizeof(float);
  NES_REQUIRE(smem <= 220 * 1024, NES_ERR_UNSUPPORTED,
              "shared_conv_pool_fwd: %zu B of feature maps per image do not fit in shared memory", smem);
  // Member groups per image: a block costs one round for loading the image's maps plus one round per
  // CP_WARPS members (a warp owns whole members); pick the split with the fewest rounds x waves.
  const int64_t sms = sm_count();
  int64_t best_groups = 1, best_cost = INT64_MAX;
  const int64_t max_groups = D < 65535 ? D : 65535;
  for (int64_t g = 1; g <= max_groups; ++g) {
    const int64_t per_g = ceil_div<int64_t>(D, g);
    const int64_t blocks = R * ceil_div<int64_t>(D, per_g);
    const int64_t cost = ceil_div<int64_t>(blocks, sms) * (ceil_div<int64_t>(per_g, CP_WARPS) + 1);
    if (cost < best_cost) { best_cost = cost; best_groups = g; }
    if (per_g <= CP_WARPS) break;
  }
  const int per = int(ceil_div<int64_t>(D, best_groups));
  dim3 grid((unsigned)R, (unsigned)ceil_div<int64_t>(D, per));
  cudaError_t e;
  cudaStream_t st = as_stream(stream);
#define NES_LAUNCH_SHARED_CONV_POOL(MODE, T)                                                                             \
  e = cudaFuncSetAttribute(shared_conv_pool_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "shared_conv_pool_fwd: shared memory opt-in failed: %s", cudaGetErrorString(e)); \
  shared_conv_pool_kernel<MODE><<<grid, CP_WARPS * 32, smem, st>>>(z, bias, bias_noise, pout, static_cast<T*>(y), R, D, Cout, out_sp, \
                                                                   Ho, Wo, antithetic, per)
  if (out_mode == 2) { NES_LAUNCH_SHARED_CONV_POOL(2, __nv_bfloat16); }
  else if (out_mode == 1) { NES_LAUNCH_SHARED_CONV_POOL(1, float); }
  else { NES_LAUNCH_SHARED_CONV_POOL(0, float); }
#undef NES_LAUNCH_SHARED_CONV_POOL
  return check_launch("shared_conv_pool_fwd");
}
