// Out-permuted convolution of an input that every member shares, fused with ReLU and 2x2 max-pooling.
//
// With output permutations only, member d's convolution of a shared image is
//   conv(x, W)[c] + s * conv(x, eps)[pout[d, c]] + bias[c] + s * bias_noise[d, c],
// so the two convolutions are computed once per image (one plain convolution with the stacked filter
// [W; eps]) and the per-member work is a gather, an add, the ReLU and the pooling.  A block keeps the
// feature maps of one image in shared memory (conv(x, W) channel-major, conv(x, eps) position-major) plus
// its members' noise-map indices, signs and bias terms.  A warp owns pooling windows, a lane a channel: the
// four W values of a window stay in registers while the warp walks the members, and because the channels
// of a member point at different noise maps, the four noise reads per stored value hit 32 different banks.
// Every store is a run of consecutive channels of one pooled pixel: the output is channels-last.
#include <cuda_bf16.h>
#include "common.cuh"

namespace nes {

__device__ inline float round_to_tf32(float a) {
  uint32_t u = __float_as_uint(a);
  u += 0x00000FFFu + ((u >> 13) & 1u);
  return __uint_as_float(u & 0xFFFFE000u);
}

// MODE: 0 = fp32, 1 = fp32 rounded to TF32, 2 = bf16, 3 = bf16 with image pairs interleaved by pixel,
// 4 = split bf16: hi = bf16(v) in the first half of the output, lo = bf16(v - hi) in the second half (same layout)
template <int MODE> struct OutType { typedef float type; };
template <> struct OutType<2> { typedef __nv_bfloat16 type; };
template <> struct OutType<3> { typedef __nv_bfloat16 type; };
template <> struct OutType<4> { typedef __nv_bfloat16 type; };

// what is stored at o (and, for the split form, lo_off elements further on)
template <int MODE, typename T>
__device__ __forceinline__ void store_pooled(T* o, int64_t lo_off, float v) {
  if constexpr (MODE == 4) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    *o = h;
    o[lo_off] = __float2bfloat16_rn(v - __bfloat162float(h));
  } else if constexpr (MODE >= 2) {
    *o = __float2bfloat16_rn(v);
  } else if constexpr (MODE == 1) {
    *o = round_to_tf32(v);
  } else {
    *o = v;
  }
}

__device__ __forceinline__ float pool_value(float a0, float a1, float a2, float a3, float add) {
  return fmaxf(fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)) + add, 0.f);
}

constexpr int CP_WARPS = 32;          // warps per block

template <int MODE>
__global__ void __launch_bounds__(CP_WARPS * 32) shared_conv_pool_kernel(
    const float* __restrict__ z, const float* __restrict__ bias, const float* __restrict__ bias_noise,
    const int16_t* __restrict__ pout, typename OutType<MODE>::type* __restrict__ y, int64_t R, int64_t D, int Cout, int osp,
    int Ho, int Wo, int antithetic, int members_per_block) {
  typedef typename OutType<MODE>::type out_t;
  extern __shared__ __align__(16) float smem[];
  const int hw = Ho * Wo, pitch = hw | 1, npitch = osp | 1;
  const int Hp = Ho / 2, Wp = Wo / 2, pooled = Hp * Wp;
  float* wmaps = smem;                                          // [Cout][pitch]      conv(x, W), channel-major
  float* nmaps = wmaps + size_t(Cout) * pitch;                  // [hw][npitch]       conv(x, eps), position-major
  float2* tab = reinterpret_cast<float2*>(smem + ((size_t(Cout) * pitch + size_t(hw) * npitch + 1) & ~size_t(1)));   // [members][Cout] (scale, add)
  int16_t* so_tab = reinterpret_cast<int16_t*>(tab + size_t(members_per_block) * Cout);        // [members][Cout] noise map
  const int64_t r = blockIdx.x;
  const int64_t d0 = int64_t(blockIdx.y) * members_per_block;
  const int nm = int((d0 + members_per_block < D ? d0 + members_per_block : D) - d0);
  const float sgn = anti_sign(r, R, antithetic);
  const float* zr = z + r * int64_t(Cout + osp) * hw;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int c = warp; c < Cout + osp; c += CP_WARPS) {
    if (c < Cout) for (int p = lane; p < hw; p += 32) wmaps[c * pitch + p] = zr[c * hw + p];
    else for (int p = lane; p < hw; p += 32) nmaps[p * npitch + (c - Cout)] = zr[c * hw + p];     // odd npitch: no conflicts
  }
  for (int e = threadIdx.x; e < nm * Cout; e += blockDim.x) {
    const int m = e / Cout, c = e - m * Cout;
    const int so = pout ? int(pout[(d0 + m) * Cout + c]) : c;
    so_tab[e] = int16_t(so < osp ? so : 0);
    tab[e] = make_float2(so < osp ? sgn : 0.f,
                         (bias ? bias[c] : 0.f) + (bias_noise ? sgn * bias_noise[(d0 + m) * Cout + c] : 0.f));
  }
  __syncthreads();
  const int64_t member_stride = int64_t(pooled) * Cout;
  const int64_t lo_off = R * D * member_stride;                   // split form: the lo copy follows the hi copy
  const int row = Wo * npitch;
  for (int c0 = 0; c0 < Cout; c0 += 32) {
    const int c = c0 + lane;
    const bool live = c < Cout;
    const int cc = live ? c : 0;
    const float* base = wmaps + cc * pitch;
    // a warp takes two pooling windows per pass (pp and pp + CP_WARPS): the member's table reads and the loop
    // bookkeeping are shared by the two stored values
    for (int pp = warp; pp < pooled; pp += 2 * CP_WARPS) {
      const int pq = pp + CP_WARPS;
      const bool two = pq < pooled;
      const int py = pp / Wp, px = pp - py * Wp;
      const int p00 = (2 * py) * Wo + 2 * px;
      const int qy = two ? pq / Wp : py, qx = two ? pq - qy * Wp : px;
      const int q00 = (2 * qy) * Wo + 2 * qx;
      const float b00 = base[p00], b01 = base[p00 + 1], b10 = base[p00 + Wo], b11 = base[p00 + Wo + 1];
      const float c00 = base[q00], c01 = base[q00 + 1], c10 = base[q00 + Wo], c11 = base[q00 + Wo + 1];
      // MODE 3: images b = 2q and 2q + 1 share rows, [q][pooled pixel][image][channel]; d0 and D are even there
      out_t* o = (MODE == 3) ? y + (((r * D + d0) / 2 * pooled + pp) * 2) * Cout + c
                             : y + ((r * D + d0) * pooled + pp) * Cout + c;
      const int64_t o_second = int64_t(pq - pp) * Cout * (MODE == 3 ? 2 : 1);     // from window pp to window pq
      const float* np = nmaps + p00 * npitch;
      const int nq = (q00 - p00) * npitch;
      const int16_t* sp = so_tab + cc;               // this channel's column of the member tables
      const float2* tp = tab + cc;
      const int o1 = npitch, o2 = row, o3 = row + npitch;
      const bool live2 = live && two;
#pragma unroll 2
      for (int m = 0; m < nm; ++m, o += ((MODE == 3) ? ((m & 1) ? int64_t(Cout) : 2 * member_stride - Cout) : member_stride),   // m: the member stepped to
                                 sp += Cout, tp += Cout) {
        // the 32 channels of a member point at 32 different noise maps = 32 different banks
        const float* n = np + int(*sp);
        const float2 t = *tp;
        const float v = pool_value(fmaf(t.x, n[0], b00), fmaf(t.x, n[o1], b01), fmaf(t.x, n[o2], b10),
                                   fmaf(t.x, n[o3], b11), t.y);
        const float* n2 = n + nq;
        const float w = pool_value(fmaf(t.x, n2[0], c00), fmaf(t.x, n2[o1], c01), fmaf(t.x, n2[o2], c10),
                                   fmaf(t.x, n2[o3], c11), t.y);
        if (live) store_pooled<MODE>(o, lo_off, v);
        if (live2) store_pooled<MODE>(o + o_second, lo_off, w);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Table form of the same layer.  Before the bias term, a stored value only depends on (channel c, noise map so,
// pooled pixel): pooled_max(conv(x, W)[c] + s * conv(x, eps)[so]).  With 1024 members and 32 channels an image has
// 32768 (member, channel) pairs but only Cout x (out_sp + 1) such maps, so a block first builds the table of pooled
// maps for ONE image and TB_CG channels in shared memory -- [channel][noise map, or none][pooled pixel], fp32 -- and
// then every member only looks its values up, adds its bias term, applies the ReLU, converts and stores: about six
// instructions per stored value instead of about forty (four gathered noise reads, four FMAs and the pooling per
// value).  The arithmetic is the same as in shared_conv_pool_kernel, operation for operation.  A block takes 16
// channels and half of the pooled pixels (the table of more does not fit): 16 bf16 channels are one 32-byte sector,
// and a block has to write whole sectors -- with 8 channels per block the other half of every sector arrived from
// another block much later and the bf16 forms ran 30 % slower than the kernel above.  A lane of the second phase owns
// two neighbouring channels of one pooled pixel: stores are 4 bytes (bf16 pairs) or 8 bytes wide, eight lanes per pixel.
constexpr int TB_CG = 16;         // channels per block
constexpr int TB_SPLIT = 2;       // pixel ranges per image and channel group
constexpr int TB_THREADS = 1024;

template <int MODE>
__global__ void __launch_bounds__(TB_THREADS) shared_conv_pool_table_kernel(
    const float* __restrict__ z, const float* __restrict__ bias, const float* __restrict__ bias_noise,
    const int16_t* __restrict__ pout, typename OutType<MODE>::type* __restrict__ y, int64_t R, int64_t D, int Cout, int osp,
    int Ho, int Wo, int antithetic, int members_per_block) {
  typedef typename OutType<MODE>::type out_t;
  extern __shared__ __align__(16) float table[];                  // [TB_CG][osp + 1][npix]
  const int hw = Ho * Wo;
  const int Hp = Ho / 2, Wp = Wo / 2, pooled = Hp * Wp;
  const int nslots = osp + 1;                                     // slot osp: the channel carries no noise
  const int64_t r = blockIdx.x;
  const int cbase = blockIdx.y * TB_CG;
  const int part = blockIdx.z % TB_SPLIT;                         // which range of the pooled pixels
  const int per_part = (pooled + TB_SPLIT - 1) / TB_SPLIT;
  const int pix0 = part * per_part;
  const int npix = (pix0 + per_part < pooled ? pix0 + per_part : pooled) - pix0;
  const int64_t d0 = int64_t(blockIdx.z / TB_SPLIT) * members_per_block;
  const int nm = int((d0 + members_per_block < D ? d0 + members_per_block : D) - d0);
  const float sgn = anti_sign(r, R, antithetic);
  const float* zr = z + r * int64_t(Cout + osp) * hw;
  // phase 1: the pooled maps.  p00 is even (2 * px and 2 * py * Wo are), so the window's rows are read as pairs
  // when Wo is even too
  const bool pairs = (Wo % 2 == 0) && ((reinterpret_cast<uintptr_t>(zr) & 7u) == 0) && (hw % 2 == 0);
  for (int e = threadIdx.x; e < nslots * npix; e += TB_THREADS) {
    const int so = e / npix, pl = e - so * npix;
    const int pp = pix0 + pl;
    const int py = pp / Wp, px = pp - py * Wp;
    const int p00 = (2 * py) * Wo + 2 * px;
    float n0 = 0.f, n1 = 0.f, n2 = 0.f, n3 = 0.f;
    if (so < osp) {
      const float* np = zr + size_t(Cout + so) * hw + p00;
      if (pairs) {
        const float2 a = *reinterpret_cast<const float2*>(np), b = *reinterpret_cast<const float2*>(np + Wo);
        n0 = a.x; n1 = a.y; n2 = b.x; n3 = b.y;
      } else {
        n0 = np[0]; n1 = np[1]; n2 = np[Wo]; n3 = np[Wo + 1];
      }
    }
#pragma unroll
    for (int cl = 0; cl < TB_CG; ++cl) {
      const float* wp = zr + size_t(cbase + cl) * hw + p00;
      float b0, b1, b2, b3;
      if (pairs) {
        const float2 a = *reinterpret_cast<const float2*>(wp), b = *reinterpret_cast<const float2*>(wp + Wo);
        b0 = a.x; b1 = a.y; b2 = b.x; b3 = b.y;
      } else {
        b0 = wp[0]; b1 = wp[1]; b2 = wp[Wo]; b3 = wp[Wo + 1];
      }
      table[(cl * nslots + so) * npix + pl] =
          fmaxf(fmaxf(fmaf(sgn, n0, b0), fmaf(sgn, n1, b1)), fmaxf(fmaf(sgn, n2, b2), fmaf(sgn, n3, b3)));
    }
  }
  __syncthreads();
  // phase 2: a warp takes members in turn; lane = (pixel slot, channel pair)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cp = lane & 7, ps = lane >> 3;
  const int c0 = cbase + 2 * cp;
  const int64_t member_stride = int64_t(pooled) * Cout;
  const int64_t lo_off = R * D * member_stride;                   // split form: the lo copy follows the hi copy
  const float bias0 = bias ? bias[c0] : 0.f, bias1 = bias ? bias[c0 + 1] : 0.f;
  // a member's noise-map indices and bias terms come from global memory: the next member's are requested before
  // this member's look-ups start, so that their latency is not paid per member
  auto member_terms = [&](int m, int& so0, int& so1, float& a0, float& a1) {
    const int64_t d = d0 + m;
    so0 = pout ? int(pout[d * Cout + c0]) : c0;
    so1 = pout ? int(pout[d * Cout + c0 + 1]) : c0 + 1;
    a0 = bias_noise ? bias_noise[d * Cout + c0] : 0.f;
    a1 = bias_noise ? bias_noise[d * Cout + c0 + 1] : 0.f;
  };
  int nso0 = 0, nso1 = 0;
  float na0 = 0.f, na1 = 0.f;
  if (warp < nm) member_terms(warp, nso0, nso1, na0, na1);
  for (int m = warp; m < nm; m += TB_THREADS / 32) {
    const int64_t d = d0 + m;
    int so0 = nso0, so1 = nso1;
    const float add0 = bias0 + sgn * na0, add1 = bias1 + sgn * na1;
    if (m + TB_THREADS / 32 < nm) member_terms(m + TB_THREADS / 32, nso0, nso1, na0, na1);
    if (so0 >= osp) so0 = osp;
    if (so1 >= osp) so1 = osp;
    const float* t0 = table + ((2 * cp) * nslots + so0) * npix;
    const float* t1 = table + ((2 * cp + 1) * nslots + so1) * npix;
    // MODE 3: images b = 2q and 2q + 1 share rows, [q][pooled pixel][image][channel]
    const int64_t b = r * D + d;
    out_t* o = (MODE == 3) ? y + (((b >> 1) * pooled) * 2 + (b & 1)) * Cout + c0 : y + b * member_stride + c0;
    const int64_t pix = (MODE == 3) ? 2 * int64_t(Cout) : int64_t(Cout);
    for (int pl = ps; pl < npix; pl += 4) {
      const float v0 = fmaxf(t0[pl] + add0, 0.f), v1 = fmaxf(t1[pl] + add1, 0.f);
      out_t* op = o + (pix0 + pl) * pix;
      if constexpr (MODE == 0) {
        *reinterpret_cast<float2*>(op) = make_float2(v0, v1);
      } else if constexpr (MODE == 1) {
        *reinterpret_cast<float2*>(op) = make_float2(round_to_tf32(v0), round_to_tf32(v1));
      } else {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
        *reinterpret_cast<__nv_bfloat162*>(op) = h;
        if constexpr (MODE == 4)
          *reinterpret_cast<__nv_bfloat162*>(op + lo_off) = __floats2bfloat162_rn(v0 - __low2float(h), v1 - __high2float(h));
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
  NES_REQUIRE(out_mode >= 0 && out_mode <= 4, NES_ERR_BAD_ARG,
              "shared_conv_pool_fwd: out_mode must be 0 (fp32), 1 (tf32), 2 (bf16), 3 (bf16, image pairs interleaved) or 4 (bf16 hi + lo)");
  NES_REQUIRE(out_mode != 3 || D % 2 == 0, NES_ERR_UNSUPPORTED, "shared_conv_pool_fwd: the pair layout needs an even number of members");
  if (R == 0 || D == 0 || Cout == 0 || Ho < 2 || Wo < 2) return NES_OK;
  NES_REQUIRE(z && y, NES_ERR_BAD_ARG, "shared_conv_pool_fwd: null pointer");
  NES_REQUIRE(R <= INT32_MAX && Cout <= 32767, NES_ERR_UNSUPPORTED, "shared_conv_pool_fwd: extent too large");
  const int64_t hw = int64_t(Ho) * Wo;
  cudaStream_t st = as_stream(stream);
  {
    // table form: Cout a multiple of TB_CG, the table of one channel group and pixel range within shared memory, 8-byte
    // aligned stores
    const int64_t pooled_t = int64_t(Ho / 2) * (Wo / 2);
    const size_t tbytes = size_t(TB_CG) * size_t(out_sp + 1) * size_t(ceil_div<int64_t>(pooled_t, TB_SPLIT)) * sizeof(float);
    if (Cout % TB_CG == 0 && tbytes <= 200 * 1024 && (reinterpret_cast<uintptr_t>(y) & 7u) == 0 && Cout / TB_CG <= 65535) {
      // members per block: all of them unless that leaves SMs idle
      const int64_t groups = R * (Cout / TB_CG) * TB_SPLIT;
      int64_t chunks = 1;
      while (groups * chunks < sm_count() && D / (chunks * 2) >= 64) chunks *= 2;
      const int64_t per_t = ceil_div<int64_t>(D, chunks);
      dim3 tgrid((unsigned)R, (unsigned)(Cout / TB_CG), (unsigned)(ceil_div<int64_t>(D, per_t) * TB_SPLIT));
      cudaError_t te;
#define NES_LAUNCH_SHARED_CONV_POOL_TABLE(MODE, T)                                                                       \
  te = cudaFuncSetAttribute(shared_conv_pool_table_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tbytes); \
  if (te != cudaSuccess) return fail(NES_ERR_LAUNCH, "shared_conv_pool_fwd: shared memory opt-in failed: %s", cudaGetErrorString(te)); \
  shared_conv_pool_table_kernel<MODE><<<tgrid, TB_THREADS, tbytes, st>>>(z, bias, bias_noise, pout, static_cast<T*>(y), R, D, Cout, \
                                                                        out_sp, Ho, Wo, antithetic, int(per_t))
      if (out_mode == 4) { NES_LAUNCH_SHARED_CONV_POOL_TABLE(4, __nv_bfloat16); }
      else if (out_mode == 3) { NES_LAUNCH_SHARED_CONV_POOL_TABLE(3, __nv_bfloat16); }
      else if (out_mode == 2) { NES_LAUNCH_SHARED_CONV_POOL_TABLE(2, __nv_bfloat16); }
      else if (out_mode == 1) { NES_LAUNCH_SHARED_CONV_POOL_TABLE(1, float); }
      else { NES_LAUNCH_SHARED_CONV_POOL_TABLE(0, float); }
#undef NES_LAUNCH_SHARED_CONV_POOL_TABLE
      return check_launch("shared_conv_pool_fwd(table)");
    }
  }
  const size_t limit = 220 * 1024;
  const size_t plane_bytes = ((size_t(Cout) * size_t(hw | 1) + size_t(hw) * size_t(out_sp | 1) + 1) & ~size_t(1)) * sizeof(float);
  const size_t member_bytes = size_t(Cout) * 10;                // one float2 and one int16 per channel
  NES_REQUIRE(plane_bytes + 8 * member_bytes <= limit, NES_ERR_UNSUPPORTED,
              "shared_conv_pool_fwd: %zu B of feature maps per image do not fit in shared memory", plane_bytes);
  // Members per block: a block costs about one round for loading the image's maps plus one round per
  // window pass over its members; pick the split with the fewest rounds x waves, within the table space.
  const int64_t sms = sm_count();
  const int64_t max_per = int64_t((limit - plane_bytes) / member_bytes);
  const int64_t pooled = int64_t(Ho / 2) * (Wo / 2);
  const int64_t passes = ceil_div<int64_t>(pooled, CP_WARPS) * ceil_div<int64_t>(Cout, 32);
  int64_t best_per = 1, best_cost = INT64_MAX;
  for (int64_t g = ceil_div<int64_t>(D, max_per); g <= D && g <= 65535; ++g) {
    const int64_t per_g = ceil_div<int64_t>(D, g);
    const int64_t blocks = R * ceil_div<int64_t>(D, per_g);
    const int64_t cost = ceil_div<int64_t>(blocks, sms) * (passes * per_g + 64);
    if (cost < best_cost) { best_cost = cost; best_per = per_g; }
    if (blocks >= 4 * sms) break;
  }
  int per = int(best_per);
  if (out_mode == 3 && (per & 1)) ++per;             // blocks start on even members
  const size_t smem = plane_bytes + size_t(per) * member_bytes + 16;
  dim3 grid((unsigned)R, (unsigned)ceil_div<int64_t>(D, per));
  cudaError_t e;
#define NES_LAUNCH_SHARED_CONV_POOL(MODE, T)                                                                             \
  e = cudaFuncSetAttribute(shared_conv_pool_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "shared_conv_pool_fwd: shared memory opt-in failed: %s", cudaGetErrorString(e)); \
  shared_conv_pool_kernel<MODE><<<grid, CP_WARPS * 32, smem, st>>>(z, bias, bias_noise, pout, static_cast<T*>(y), R, D, Cout, out_sp, \
                                                                   Ho, Wo, antithetic, per)
  if (out_mode == 4) { NES_LAUNCH_SHARED_CONV_POOL(4, __nv_bfloat16); }
  else if (out_mode == 3) { NES_LAUNCH_SHARED_CONV_POOL(3, __nv_bfloat16); }
  else if (out_mode == 2) { NES_LAUNCH_SHARED_CONV_POOL(2, __nv_bfloat16); }
  else if (out_mode == 1) { NES_LAUNCH_SHARED_CONV_POOL(1, float); }
  else { NES_LAUNCH_SHARED_CONV_POOL(0, float); }
#undef NES_LAUNCH_SHARED_CONV_POOL
  return check_launch("shared_conv_pool_fwd");
}
