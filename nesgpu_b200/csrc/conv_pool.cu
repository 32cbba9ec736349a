// Out-permuted convolution of an input that every member shares, fused with ReLU and 2x2 max-pooling.
//
// With output permutations only, member d's convolution of a shared image is
//   conv(x, W)[c] + s * conv(x, eps)[pout[d, c]] + bias[c] + s * bias_noise[d, c],
// so the two convolutions are computed once per image (one plain convolution with the stacked filter
// [W; eps]) and the per-member work is a gather, an add, the ReLU and the pooling.  A block keeps the
// stacked feature maps of one image in shared memory (plane pitch odd, so lanes that hold different
// channels hit different banks) and walks a group of members; lanes are channels, so every store is a
// run of consecutive channels of one pooled pixel: the output is channels-last.
#include "common.cuh"

namespace nes {

__device__ inline float round_to_tf32(float a) {
  uint32_t u = __float_as_uint(a);
  u += 0x00000FFFu + ((u >> 13) & 1u);
  return __uint_as_float(u & 0xFFFFE000u);
}

__global__ void __launch_bounds__(512) shared_conv_pool_kernel(
    const float* __restrict__ z, const float* __restrict__ bias, const float* __restrict__ bias_noise,
    const int16_t* __restrict__ pout, float* __restrict__ y, int64_t R, int64_t D, int Cout, int osp,
    int Ho, int Wo, int antithetic, int round_tf32, int members_per_block) {
  extern __shared__ float planes[];                 // (Cout + osp) planes of Ho*Wo (+1 pad) floats
  const int hw = Ho * Wo, pitch = hw | 1;
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
      float* out = y + ((r * D + d) * pooled) * Cout + c;
      for (int py = 0; py < Hp; ++py) {
        const int row = (2 * py) * Wo;
#pragma unroll 4
        for (int px = 0; px < Wp; ++px) {
          const int p00 = row + 2 * px;
          const float v0 = base[p00] + s * noise[p00];
          const float v1 = base[p00 + 1] + s * noise[p00 + 1];
          const float v2 = base[p00 + Wo] + s * noise[p00 + Wo];
          const float v3 = base[p00 + Wo + 1] + s * noise[p00 + Wo + 1];
          float v = fmaxf(fmaxf(fmaxf(v0, v1), fmaxf(v2, v3)) + add, 0.f);
          if (round_tf32) v = round_to_tf32(v);
          if (live) out[int64_t(py * Wp + px) * Cout] = v;
        }
      }
    }
  }
}

}  // namespace nes

using namespace nes;

extern "C" int nes_shared_conv_pool_fwd(const float* z, const float* bias, const float* bias_noise,
                                        const int16_t* pout, float* y, int64_t R, int64_t D, int Cout, int out_sp,
                                        int Ho, int Wo, int antithetic, int round_tf32, nes_stream_t stream) {
  NES_REQUIRE(R >= 0 && D >= 0 && Cout >= 0 && out_sp >= 0 && Ho >= 0 && Wo >= 0, NES_ERR_BAD_ARG,
              "shared_conv_pool_fwd: negative extent");
  NES_REQUIRE(out_sp <= Cout, NES_ERR_BAD_ARG, "shared_conv_pool_fwd: out_sp exceeds the channel count");
  if (R == 0 || D == 0 || Cout == 0 || Ho < 2 || Wo < 2) return NES_OK;
  NES_REQUIRE(z && y, NES_ERR_BAD_ARG, "shared_conv_pool_fwd: null pointer");
  NES_REQUIRE(R <= INT32_MAX, NES_ERR_UNSUPPORTED, "shared_conv_pool_fwd: too many images");
  const int64_t hw = int64_t(Ho) * Wo;
  const size_t smem = size_t(Cout + out_sp) * size_t(hw | 1) * sizeof(float);
  NES_REQUIRE(smem <= 220 * 1024, NES_ERR_UNSUPPORTED,
              "shared_conv_pool_fwd: %zu B of feature maps per image do not fit in shared memory", smem);
  cudaError_t e = cudaFuncSetAttribute(shared_conv_pool_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "shared_conv_pool_fwd: shared memory opt-in failed: %s", cudaGetErrorString(e));
  // member groups per image so that the grid is just under a whole number of waves (one block per SM),
  // at least 8 members per block
  int64_t groups = (int64_t(sm_count()) * 2) / R;
  if (groups < 1) groups = ceil_div<int64_t>(sm_count(), R);
  if (groups > ceil_div<int64_t>(D, 8)) groups = ceil_div<int64_t>(D, 8);
  if (groups < 1) groups = 1;
  if (groups > 65535) groups = 65535;
  const int per = int(ceil_div<int64_t>(D, groups));
  dim3 grid((unsigned)R, (unsigned)ceil_div<int64_t>(D, per));
  shared_conv_pool_kernel<<<grid, 512, smem, as_stream(stream)>>>(z, bias, bias_noise, pout, y, R, D, Cout, out_sp, Ho, Wo,
                                                                  antithetic, round_tf32, per);
  return check_launch("shared_conv_pool_fwd");
}
