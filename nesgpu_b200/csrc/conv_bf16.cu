// Tensor-core convolution for the per-member layers, BF16 mode, with the filter as the M operand.
//
// Same decomposition as the TF32 kernel in conv_tc.cu -- persistent thread blocks over (member, sign)
// units, the member's effective filter W_d = W + s * E_d built in shared memory, the input read from a
// zero-padded, channel-chunked, pre-swizzled copy by one bulk async copy per (tile, chunk), filter taps
// realised as row offsets into the staged run -- but arranged so that one tcgen05.mma does four times
// the work, because with N = Cout = 64 the TF32 kernel is bound by the number of MMA instructions:
//   * operands are bf16: one 128-byte swizzle row holds 64 channels and one instruction covers K = 16;
//   * the product is transposed: D[Cout x pixels] = W_d[Cout x K] . X[pixels x K]^T, i.e. the filter is
//     the A operand (M = 64 or 128 rows) and the staged pixel run is the B operand with N = 256 pixels.
// An accumulator tile is M TMEM lanes x 256 fp32 columns; two of them (all 512 columns) alternate
// between the MMA issuer and the epilogue.  With M = 64 the accumulator occupies lanes 0-15 of each
// 32-lane quadrant, so each epilogue warp reads its quadrant with tcgen05.ld.32x32b, its first 16 threads
// own one output channel each, and a per-warp shared-memory transpose turns that into stores of 32
// consecutive positions of one channel plane.  All eight builder warps drain (two per lane quadrant).
// Reduced precision (bf16 operands, fp32 accumulation): a stated mode, relative error ~3e-3.
//
// TERMS = 3 is the split form that holds the fp32 bar on the same tensor-core path: both operands are split
// into two bf16 parts, v = hi + lo + O(2^-18 |v|) with hi = bf16(v), lo = bf16(v - hi), and the accumulator
// takes W_hi.x_hi + W_lo.x_hi + W_hi.x_lo (the dropped W_lo.x_lo term is of the same order as the
// residuals): relative error of a few 1e-6.  The filter builders write W_d twice (hi and lo copies of the
// same layout), the layout pre-pass writes x twice, and per (tile, channel chunk) the producer fetches the
// hi run and the lo run into two consecutive pipeline slots; tiles are 128 positions wide so that two slots
// of each kind fit next to the two filter copies.  Permuted-noise layers with 64 input channels and at most 64 output
// channels take the tensor-memory form of this product instead (conv_split_tmem_kernel below).
#include <cuda_bf16.h>
#include "tc_ptx.cuh"

namespace nes {

int launch_permuted_maps(const int16_t* pin, const int16_t* pout, int16_t* omap, int16_t* imap, int64_t D,
                         int Cin, int Cout, int in_sp, int out_sp, cudaStream_t st);

namespace tc {

constexpr int BF_THREADS = 320;     // producer, MMA issuer, 4 epilogue + builder warps, 4 builder warps
constexpr int BF_NT = 256;          // pixels (positions) per tile = MMA N (one-term form)
constexpr int BF_NT3 = 128;         // the same for the three-term form

struct ConvBfParams {
  int Cin, H, W, Cout, kh, kw, ph, pw, dh, dw, Ho, Wo;
  int Hp, Wp, tiles_img, img_rows, load_bytes, stage_bytes;
  int M;                         // 64 or 128 filter rows in the MMA (rows >= Cout are zero)
  long long D, R;
  int antithetic, sign_groups, units;
  int stages, kchunks, cchunks;
  long long lo_offset;           // three-term form: element offset of the lo copy of the staged input
  int tmem_filter;               // three-term form with the stacked [W_hi; W_lo] filter in tensor memory (conv_split_tmem_kernel)
  int eps_rows, e_pitch;         // that form: rows of the shared noise kept in shared memory and their pitch in bytes
  const float* weight; const float* bias; const float* bias_noise; float* y;
  int noise_kind;                // 1 dense (D,Cout,Cin,ksz), 2 permuted (out_sp,in_sp,ksz) through omap / imap
  const float* noise; const int16_t* omap; const int16_t* imap; int in_sp;
  const float* weight_t; const float* noise_t;    // (n, tap, c) re-ordered fp32 copies for noise_kind 2
  int identity_in;
  int dense_vec;                 // dense noise: weight and noise are 16-byte aligned (vector path of the filter build)
};

__device__ __forceinline__ void bf_unit_range(const ConvBfParams& p, int sg, long long& r0, long long& r1, float& s) {
  if (!p.antithetic) { r0 = 0; r1 = p.R; s = 1.f; return; }
  const long long half = (p.R + 1) / 2;
  if (sg == 0) { r0 = 0; r1 = half; s = 1.f; } else { r0 = half; r1 = p.R; s = -1.f; }
}

__device__ __forceinline__ void mma_bf16_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "mov.b64 da, {%1, %3};\n"
      "mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n"
      "}\n"
      ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// hi = bf16(v), lo = bf16(v - hi)
__device__ __forceinline__ void split_bf16(float v, float& hi, float& lo) {
  hi = __bfloat162float(__float2bfloat16_rn(v));
  lo = v - hi;
}

// Optional timeline (build with -DNES_CONV_TRACE): block 0 writes %globaltimer (ns) into slot [tile * 16 + phase]
// for its first 64 tiles (phases 0-1 producer, 2-6 MMA issuer, 7-8 epilogue, 9-10 filter build of the tile's member).
#ifdef NES_CONV_TRACE
__device__ long long g_conv_trace[64 * 16];
__device__ __forceinline__ void conv_trace(uint32_t tile, int phase) {
  if (blockIdx.x == 0 && tile < 64) {
    long long tns;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tns));
    g_conv_trace[tile * 16 + phase] = tns;
  }
}
#define CONV_TRACE(cond, tile, phase) do { if (cond) conv_trace(tile, phase); } while (0)
#else
#define CONV_TRACE(cond, tile, phase) do { } while (0)
#endif

template <int TERMS, int NT>
__global__ void __launch_bounds__(BF_THREADS, 1) conv_bf16_kernel(const __nv_bfloat16* __restrict__ xs, const ConvBfParams p) {
  extern __shared__ unsigned char dyn_raw[];
  const unsigned int timeouts_at_start = timeouts_so_far();
  const uint32_t raw = smem_u32(dyn_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  unsigned char* wd = dyn_raw + pad;                                   // [kchunks][M][128 B] (x 2 with TERMS == 3: hi, lo)
  const int wd_chunk_bytes = p.M * 128;
  const size_t wd_copy_bytes = size_t(p.kchunks) * wd_chunk_bytes;
  const size_t lo_off = wd_copy_bytes;                                 // from a hi filter element to its lo partner
  unsigned char* stages_base = wd + (TERMS == 3 ? 2 : 1) * wd_copy_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(stages_base + size_t(p.stages) * p.stage_bytes);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;     // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint64_t* wd_ready = acc_empty + 2;
  uint64_t* wd_free = wd_ready + 1;
  uint64_t* tbl_ready = wd_free + 1;
  uint64_t* stage_bar = tbl_ready + 1;       // dense filter build: all eight builder warps have reached the same point
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stage_bar + 1);
  const int table_maps_bytes = ((2 * (p.Cout + p.Cin)) + 15) & ~15;
  const int table_bytes = table_maps_bytes + 4 * p.Cout;
  unsigned char* tables = reinterpret_cast<unsigned char*>(tmem_slot) + 16;
  // [8 warps][rows per warp][33] epilogue transpose (8 bytes per tap of spare room lie in front of it)
  float* xpose = reinterpret_cast<float*>(tables + 2 * size_t(table_bytes) + 8 * size_t(p.kh) * p.kw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ksz = p.kh * p.kw;
  const int K = p.Cin * ksz;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    mbar_init(wd_ready, 8);
    mbar_init(wd_free, 1);
    mbar_init(tbl_ready, 8);
    mbar_init(stage_bar, 8);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // filter rows beyond Cout (padding up to M) stay zero for the whole kernel
  if (p.M > p.Cout) {
    for (int e = threadIdx.x; e < p.kchunks * (p.M - p.Cout) * 8; e += BF_THREADS) {
      const int jc = e / ((p.M - p.Cout) * 8);
      const int r = e - jc * (p.M - p.Cout) * 8;
      const int n = p.Cout + r / 8, g16 = r & 7;
      const size_t off = size_t(jc) * wd_chunk_bytes + (n >> 3) * 1024 + (n & 7) * 128 + (g16 << 4);
      *reinterpret_cast<uint4*>(wd + off) = make_uint4(0, 0, 0, 0);
      if (TERMS == 3) *reinterpret_cast<uint4*>(wd + wd_copy_bytes + off) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, uint32_t(2 * NT));
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ producer: one bulk copy per (tile, chunk)
      uint32_t g = 0, tt = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        const long long d = u / p.sign_groups;
        long long r0, r1; float s;
        bf_unit_range(p, u % p.sign_groups, r0, r1, s);
        for (long long r = r0; r < r1 && ok; ++r) {
          const long long b = r * p.D + d;
          for (int ti = 0; ti < p.tiles_img && ok; ++ti, ++tt)
            for (int cc = 0; cc < p.cchunks; ++cc, ++g) {
              const int st = g % p.stages;
              const uint32_t phs = (g / p.stages) & 1;
              if (!mbar_wait(&empty[st], phs ^ 1, 1)) { ok = false; break; }
              CONV_TRACE(cc == 0, tt, 0);
              const long long row0 = (b * p.cchunks + cc) * (long long)p.img_rows + (long long)ti * NT;
              mbar_expect_tx(&full[st], uint32_t(p.load_bytes));
              bulk_load_1d(stages_base + size_t(st) * p.stage_bytes, xs + row0 * 64, uint32_t(p.load_bytes), &full[st]);
              if (TERMS == 3) {
                // the lo run of the same positions goes into the next pipeline slot
                ++g;
                const int st2 = g % p.stages;
                const uint32_t phs2 = (g / p.stages) & 1;
                if (!mbar_wait(&empty[st2], phs2 ^ 1, 1)) { ok = false; break; }
                CONV_TRACE(cc == 0, tt, 1);
                mbar_expect_tx(&full[st2], uint32_t(p.load_bytes));
                bulk_load_1d(stages_base + size_t(st2) * p.stage_bytes, xs + p.lo_offset + row0 * 64, uint32_t(p.load_bytes), &full[st2]);
              }
            }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer: the whole warp runs this loop in
    // converged control flow and one elected lane issues each instruction (see warp_mma_bf16)
    // D = fp32, A = B = bf16, both K-major, N = NT positions, M = filter rows
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(NT >> 3) << 17) | (uint32_t(p.M >> 4) << 24);
    const uint64_t desc0 = smem_desc_sw128(0);
    const uint64_t wd_desc = desc0 + uint64_t(smem_u32(wd) >> 4);
    const uint32_t cc_step = uint32_t(wd_chunk_bytes >> 4);
    const uint32_t tap_step = uint32_t(p.cchunks) * cc_step;            // filter chunks of one tap
    const uint32_t wd_copy_units = uint32_t(wd_copy_bytes >> 4);        // from the hi filter copy to the lo copy
    uint32_t g = 0, t = 0, ul = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      long long r0, r1; float s;
      bf_unit_range(p, u % p.sign_groups, r0, r1, s);
      if (r1 <= r0) continue;
      if (!warp_mbar_wait(wd_ready, ul & 1, 2)) { ok = false; break; }
      tc_fence_after();
      const long long ntiles = (r1 - r0) * p.tiles_img;
      for (long long ti = 0; ti < ntiles && ok; ++ti, ++t) {
        const uint32_t buf = t & 1;
        if (!warp_mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, 2)) { ok = false; break; }
        tc_fence_after();
        CONV_TRACE(lane == 0, t, 2);
        const uint32_t tmem_d = tmem_base + buf * uint32_t(NT);
        for (int cc = 0; cc < p.cchunks; ++cc, ++g) {
          const int st = g % p.stages;
          const uint32_t phs = (g / p.stages) & 1;
          if (!warp_mbar_wait(&full[st], phs, 2)) { ok = false; break; }
          tc_fence_after();
          CONV_TRACE(lane == 0 && cc == 0, t, 3);
          const uint64_t x_desc = desc0 + uint64_t(smem_u32(stages_base + size_t(st) * p.stage_bytes) >> 4);
          const uint64_t w_desc = wd_desc + uint64_t(uint32_t(cc) * cc_step);
          uint32_t accumulate = (cc > 0) ? 1u : 0u;
          for (int i = 0, tap = 0; i < p.kh; ++i)
            for (int j = 0; j < p.kw; ++j, ++tap) {
              // pixel-row shift of the tap in 16-byte units (8 per 128-byte row); the tap's filter chunk
              const uint64_t bl = x_desc + uint64_t(uint32_t(i * p.dh * p.Wp + j * p.dw) * 8u);
              const uint64_t al = w_desc + uint64_t(uint32_t(tap) * tap_step);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                warp_mma_bf16(tmem_d, al + uint64_t(2 * k), bl + uint64_t(2 * k), idesc, accumulate);
                accumulate = 1u;
                // W_lo . x_hi on the same staged run
                if (TERMS == 3) warp_mma_bf16(tmem_d, al + uint64_t(wd_copy_units + 2 * k), bl + uint64_t(2 * k), idesc, 1u);
              }
            }
          warp_mma_commit(&empty[st]);
          CONV_TRACE(lane == 0 && cc == 0, t, 4);
          if (TERMS == 3) {
            // W_hi . x_lo: the lo run sits in the next slot
            ++g;
            const int st2 = g % p.stages;
            const uint32_t phs2 = (g / p.stages) & 1;
            if (!warp_mbar_wait(&full[st2], phs2, 2)) { ok = false; break; }
            tc_fence_after();
            CONV_TRACE(lane == 0 && cc == 0, t, 5);
            const uint64_t x2 = desc0 + uint64_t(smem_u32(stages_base + size_t(st2) * p.stage_bytes) >> 4);
            for (int i = 0, tap = 0; i < p.kh; ++i)
              for (int j = 0; j < p.kw; ++j, ++tap) {
                const uint64_t bl = x2 + uint64_t(uint32_t(i * p.dh * p.Wp + j * p.dw) * 8u);
                const uint64_t al = w_desc + uint64_t(uint32_t(tap) * tap_step);
#pragma unroll
                for (int k = 0; k < 4; ++k) warp_mma_bf16(tmem_d, al + uint64_t(2 * k), bl + uint64_t(2 * k), idesc, 1u);
              }
            warp_mma_commit(&empty[st2]);
            CONV_TRACE(lane == 0 && cc == 0, t, 6);
          }
        }
        warp_mma_commit(&acc_full[buf]);
      }
      warp_mma_commit(wd_free);
      ++ul;
    }
  } else {
    // ---------------------------------------------------------------------- filter builders / epilogue
    const int bt = threadIdx.x - 64;            // builder thread 0..255
    const int q = warp & 3;
    // accumulator row (= output channel) this thread reads: with M = 128 lane i of quadrant q is row 32q+i;
    // with M = 64 rows 16q .. 16q+15 sit in the first 16 lanes of quadrant q
    const int chan = (p.M == 128) ? (q * 32 + lane) : (q * 16 + lane);
    const bool lane_has_row = (p.M == 128) || (lane < 16);
    const int HoWo = p.Ho * p.Wo;
    const int k8 = K / 8, c8n = p.Cin / 8;
    uint32_t t = 0, ul = 0, n_stage_sync = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      const long long d = u / p.sign_groups;
      long long r0, r1; float s;
      bf_unit_range(p, u % p.sign_groups, r0, r1, s);
      if (r1 <= r0) continue;
      unsigned char* tb = tables + size_t(ul & 1) * table_bytes;
      int16_t* omap_s = reinterpret_cast<int16_t*>(tb);
      int16_t* imap_s = omap_s + p.Cout;
      float* add_s = reinterpret_cast<float*>(tb + table_maps_bytes);
      for (int n = bt; n < p.Cout; n += 256) {
        omap_s[n] = (p.noise_kind == 2) ? p.omap[d * p.Cout + n] : int16_t(n);
        float a = p.bias ? __ldg(p.bias + n) : 0.f;
        if (p.bias_noise) a += s * __ldg(p.bias_noise + d * p.Cout + n);
        add_s[n] = a;
      }
      for (int c = bt; c < p.Cin; c += 256) imap_s[c] = (p.noise_kind == 2) ? p.imap[d * p.Cin + c] : int16_t(c);
      __syncwarp();
      if (lane == 0) mbar_arrive(tbl_ready);
      if (!mbar_wait_relaxed(tbl_ready, ul & 1, 4)) { ok = false; break; }
      if (!mbar_wait_relaxed(wd_free, (ul & 1) ^ 1, 4)) { ok = false; break; }
      CONV_TRACE(threadIdx.x == 128, t, 9);

      if (p.noise_kind == 1 && ksz == 9 && p.dense_vec) {
        // dense member noise in its native (n, c, tap) order, 3x3 filters.  The filter W + s E_d is formed element by
        // element in stream order (W has the same order): coalesced 16-byte loads, 1008 of them per round, the sums
        // parked in the epilogue's transpose buffers (idle during the build).  After a block-wide hand-over a thread
        // takes four consecutive channels of one filter row = 36 consecutive floats from there (conflict-free at a
        // 144-byte stride); with the loops unrolled every element's tap and channel are compile-time constants, and
        // the four channels of a tap go to the filter image as one 8-byte store per copy.  (Reading the 36 floats
        // straight from global memory made every load instruction touch 36 lines: 16-20 us per member.)
        constexpr int QR = 112;                                  // quads (of 9 float4) per round
        const int quads_per_row = p.Cin >> 2;
        const int nquads = p.Cout * quads_per_row;
        const int total4 = nquads * 9;
        const float4* W4 = reinterpret_cast<const float4*>(p.weight);
        const float4* E4 = reinterpret_cast<const float4*>(p.noise + size_t(d) * p.Cout * K);
        float4* staging = reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(xpose) + ((16u - (smem_u32(xpose) & 15u)) & 15u));
        auto block_sync = [&]() -> bool {
          __syncwarp();
          if (lane == 0) mbar_arrive(stage_bar);
          const bool done = mbar_wait(stage_bar, n_stage_sync & 1, 4);
          ++n_stage_sync;
          return __all_sync(0xffffffffu, done ? 1 : 0) != 0;
        };
        float4 wv[4], ev[4];
        auto fetch = [&](int base4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int idx = base4 + bt + 256 * i;
            const bool in = bt + 256 * i < QR * 9 && idx < total4;
            wv[i] = in ? __ldg(W4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
            ev[i] = in ? __ldcs(E4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        };
        fetch(0);
        // the buffers may still serve another warp's epilogue of the previous member: everybody arrives here first
        bool fine = block_sync();
        for (int q0 = 0; q0 < nquads && fine; q0 += QR) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int li = bt + 256 * i;
            if (li < QR * 9)
              staging[li] = make_float4(fmaf(s, ev[i].x, wv[i].x), fmaf(s, ev[i].y, wv[i].y), fmaf(s, ev[i].z, wv[i].z),
                                        fmaf(s, ev[i].w, wv[i].w));
          }
          if (q0 + QR < nquads) fetch((q0 + QR) * 9);            // the next round's loads travel during this round
          if (!block_sync()) { fine = false; break; }
          const int quad = q0 + bt;
          if (bt < QR && quad < nquads) {
            const int n = quad / quads_per_row, c0 = (quad - n * quads_per_row) * 4;
            float f[36];
#pragma unroll
            for (int i = 0; i < 9; ++i) {
              const float4 v = staging[bt * 9 + i];
              f[4 * i] = v.x; f[4 * i + 1] = v.y; f[4 * i + 2] = v.z; f[4 * i + 3] = v.w;
            }
            unsigned char* rowp = wd + (n >> 3) * 1024 + (n & 7) * 128;
#pragma unroll
            for (int tap = 0; tap < 9; ++tap) {
              const int kk = tap * p.Cin + c0;                 // element j of the run is channel j / 9, tap j % 9
              const int jc = kk >> 6, col = kk & 63;
              unsigned char* dst = rowp + size_t(jc) * wd_chunk_bytes + ((((col >> 3) ^ (n & 7))) << 4) + (col & 7) * 2;
              const float v0 = f[tap], v1 = f[9 + tap], v2 = f[18 + tap], v3 = f[27 + tap];
              const uint32_t p01 = pack_bf16(v0, v1), p23 = pack_bf16(v2, v3);
              *reinterpret_cast<uint2*>(dst) = make_uint2(p01, p23);
              if (TERMS == 3)
                *reinterpret_cast<uint2*>(dst + lo_off) =
                    make_uint2(pack_bf16(v0 - __uint_as_float(p01 << 16), v1 - __uint_as_float(p01 & 0xffff0000u)),
                               pack_bf16(v2 - __uint_as_float(p23 << 16), v3 - __uint_as_float(p23 & 0xffff0000u)));
            }
          }
          if (!block_sync()) { fine = false; break; }            // the staging area is free again
        }
        if (!fine) { ok = false; break; }
      } else if (p.noise_kind == 1) {
        // dense member noise in its native (n, c, tap) order: coalesced reads, scattered 2-byte writes
        const int total = p.Cout * K;
        const float* E = p.noise + size_t(d) * total;
        for (int base = bt; base < total; base += 256 * 8) {
          float wv[8], ev[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int idx = base + i * 256;
            wv[i] = idx < total ? __ldg(p.weight + idx) : 0.f;
            ev[i] = idx < total ? __ldcs(E + idx) : 0.f;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int idx = base + i * 256;
            if (idx >= total) break;
            const int n = idx / K;
            const int rem = idx - n * K;
            const int c = rem / ksz, tap = rem - c * ksz;
            const int kk = tap * p.Cin + c;
            const int jc = kk >> 6, col = kk & 63;
            unsigned char* dst = wd + size_t(jc) * wd_chunk_bytes + (n >> 3) * 1024 + (n & 7) * 128 +
                                 ((((col >> 3) ^ (n & 7))) << 4) + (col & 7) * 2;
            const float v = fmaf(s, ev[i], wv[i]);
            const __nv_bfloat16 vh = __float2bfloat16_rn(v);
            *reinterpret_cast<__nv_bfloat16*>(dst) = vh;
            if (TERMS == 3) *reinterpret_cast<__nv_bfloat16*>(dst + lo_off) = __float2bfloat16_rn(v - __bfloat162float(vh));
          }
        }
      } else {
        // W and eps re-ordered to (n, tap, c): eight consecutive channels = one 16-byte bf16 group
        const float4* Wt = reinterpret_cast<const float4*>(p.weight_t);
        const bool identity_in = p.identity_in != 0;
        const int groups = p.Cout * k8;
        const int step_n = 256 / k8, step_r = 256 - step_n * k8;
        int n_cur = bt / k8, r_cur = bt - n_cur * k8;
        constexpr int BATCH = 3;
        for (int g0 = bt; g0 < groups; g0 += 256 * BATCH) {
          float4 wa[BATCH], wb[BATCH], ea[BATCH], eb[BATCH];
          int nn[BATCH], kk[BATCH];
#pragma unroll
          for (int i = 0; i < BATCH; ++i) {
            const int gidx = g0 + i * 256;
            wa[i] = make_float4(0.f, 0.f, 0.f, 0.f); wb[i] = wa[i]; ea[i] = wa[i]; eb[i] = wa[i]; nn[i] = -1; kk[i] = 0;
            if (gidx < groups) {
              const int n = n_cur, rem = r_cur;
              const int tap = rem / c8n, c = (rem - tap * c8n) * 8;
              nn[i] = n; kk[i] = tap * p.Cin + c;
              wa[i] = __ldg(Wt + 2 * size_t(gidx));
              wb[i] = __ldg(Wt + 2 * size_t(gidx) + 1);
              const int so = (p.noise_kind == 2) ? int(omap_s[n]) : -1;
              if (so >= 0) {
                const float* er = p.noise_t + (size_t(so) * ksz + tap) * p.in_sp;
                if (identity_in) {
                  ea[i] = __ldg(reinterpret_cast<const float4*>(er + c));
                  eb[i] = __ldg(reinterpret_cast<const float4*>(er + c) + 1);
                } else {
                  float e8[8];
#pragma unroll
                  for (int z = 0; z < 8; ++z) { const int ci = imap_s[c + z]; e8[z] = ci >= 0 ? __ldg(er + ci) : 0.f; }
                  ea[i] = make_float4(e8[0], e8[1], e8[2], e8[3]);
                  eb[i] = make_float4(e8[4], e8[5], e8[6], e8[7]);
                }
              }
            }
            n_cur += step_n; r_cur += step_r;
            if (r_cur >= k8) { r_cur -= k8; ++n_cur; }
          }
#pragma unroll
          for (int i = 0; i < BATCH; ++i) {
            if (nn[i] < 0) continue;
            const int n = nn[i];
            const int jc = kk[i] >> 6, col = kk[i] & 63;
            unsigned char* dst = wd + size_t(jc) * wd_chunk_bytes + (n >> 3) * 1024 + (n & 7) * 128 +
                                 ((((col >> 3) ^ (n & 7))) << 4);
            const float f[8] = {fmaf(s, ea[i].x, wa[i].x), fmaf(s, ea[i].y, wa[i].y), fmaf(s, ea[i].z, wa[i].z), fmaf(s, ea[i].w, wa[i].w),
                                fmaf(s, eb[i].x, wb[i].x), fmaf(s, eb[i].y, wb[i].y), fmaf(s, eb[i].z, wb[i].z), fmaf(s, eb[i].w, wb[i].w)};
            if (TERMS == 3) {
              float h[8], l[8];
#pragma unroll
              for (int z = 0; z < 8; ++z) split_bf16(f[z], h[z], l[z]);
              *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16(h[0], h[1]), pack_bf16(h[2], h[3]), pack_bf16(h[4], h[5]), pack_bf16(h[6], h[7]));
              *reinterpret_cast<uint4*>(dst + lo_off) = make_uint4(pack_bf16(l[0], l[1]), pack_bf16(l[2], l[3]), pack_bf16(l[4], l[5]), pack_bf16(l[6], l[7]));
            } else {
              *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
            }
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(wd_ready);
      CONV_TRACE(threadIdx.x == 128, t, 10);

      {
        // Epilogue (all eight builder warps; two warps share a TMEM lane quadrant and split the tile's columns
        // between them): a thread holds one output channel (accumulator row) and 32 consecutive positions per
        // tcgen05.ld; the warp transposes that 32-position chunk through shared memory so that each store
        // instruction writes 32 consecutive positions of ONE channel plane (full 128-byte lines).
        const bool owns = lane_has_row && chan < p.Cout;
        const float add = owns ? add_s[chan] : 0.f;
        const int rows_per_warp = (p.M == 128) ? 32 : 16;
        const int chan0 = (p.M == 128) ? q * 32 : q * 16;
        float* xp = xpose + size_t(warp - 2) * rows_per_warp * 33;
        const int col_lo = (warp < 6) ? 0 : NT / 2, col_hi = col_lo + NT / 2;
        for (long long r = r0; r < r1 && ok; ++r) {
          const long long b = r * p.D + d;
          float* img = p.y + size_t(b) * p.Cout * HoWo;
          for (int ti = 0; ti < p.tiles_img && ok; ++ti, ++t) {
            const uint32_t buf = t & 1;
            if (!mbar_wait_relaxed(&acc_full[buf], (t >> 1) & 1, 3)) { ok = false; break; }
            tc_fence_after();
            const bool live = (timeouts_so_far() == timeouts_at_start);
            for (int c0 = col_lo; c0 < col_hi; c0 += 32) {
              uint32_t acc[32];
              tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + buf * uint32_t(NT) + uint32_t(c0), acc);
              if (lane_has_row) {
#pragma unroll
                for (int j = 0; j < 32; ++j) xp[lane * 33 + j] = __uint_as_float(acc[j]) + add;
              }
              __syncwarp();
              const int qpos = ti * NT + c0 + lane;
              const int oy = qpos / p.Wp, ox = qpos - oy * p.Wp;
              if (live && oy < p.Ho && ox < p.Wo) {
                float* dst = img + size_t(chan0) * HoWo + oy * p.Wo + ox;
                for (int rl = 0; rl < rows_per_warp && chan0 + rl < p.Cout; ++rl) dst[size_t(rl) * HoWo] = xp[rl * 33 + lane];
              }
              __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
          }
        }
      }
      ++ul;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, uint32_t(2 * NT));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Split-bf16 convolution with the member filter in TENSOR MEMORY (permuted-noise layers, Cin = 64, at most 64 output
// channels, at most 9 taps).  The two bf16 parts of the filter are stacked into one M = 128 operand (rows 0-63 = W_hi,
// rows 64-127 = W_lo of the same channels), so two MMAs per K step (on x_hi and on x_lo) give all four partial
// products, and that operand lives in tensor memory: lane = filter row, 8 columns (16 bf16) per K step, 36 K steps =
// 288 columns next to two accumulators of SP_NT = 96 columns.  An MMA then reads only its B operand (the staged
// positions) from shared memory.  With both operands in shared memory an M = 128, N = 128 instruction needs the
// whole shared-memory bandwidth (8 KB per 64 cycles), and the bulk copies and the epilogue's transposes compete
// for it: measured 4.3 us per 128-position tile against 2.9 us of tensor-pipe time.  Shared memory now only holds
// the input pipeline (up to 8 slots), the per-member tables and the epilogue's exchange buffers.
//
// Roles as in conv_bf16_kernel.  The eight builder warps write the filter with tcgen05.st: the thread of tensor-memory
// lane r forms W_d[r mod 64, :] = W + s * eps[omap] for 32 channels of one tap at a time and keeps its hi or its lo
// part; the two warps of a lane quadrant take half of the (tap, channel half) groups each.  Where the values come
// from: the shared noise eps (out_sp rows, the same for every member; a member only chooses which row goes where)
// is copied into shared memory once per block, and the 32 x 32 W tile of a group arrives by one TMA tile load into
// a ring of three tiles per warp pair (the warp of rows c and the warp of rows c + 64 read the same tile), issued
// three groups ahead and across member boundaries.  Plain loads were tried first: a warp gets one 512-byte load
// instruction through every ~90 cycles (measured), which made the build 13 us per member.  Epilogue: accumulator
// rows c and c + 64 are added by the two warps (lane quadrants q and q + 2) that share a column half; each writes the
// 16-column chunks it does not finish into its partner's buffer, adds what the partner wrote into its own, transposes
// there and stores 16 consecutive positions of two channel planes per instruction.  A half has three chunks: each
// warp finishes one, the third alternates between them from tile to tile.
constexpr int SP_NT = 96;
constexpr int SP_A_COL = 224;          // first tensor-memory column of the filter operand
constexpr int SP_WRING = 3;            // W tiles in flight per builder warp pair

__global__ void __launch_bounds__(BF_THREADS, 1) conv_split_tmem_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                        const __nv_bfloat16* __restrict__ xs, const ConvBfParams p) {
  constexpr int NT = SP_NT;
  extern __shared__ unsigned char dyn_raw[];
  const unsigned int timeouts_at_start = timeouts_so_far();
  const uint32_t raw = smem_u32(dyn_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  unsigned char* stages_base = dyn_raw + pad;
  unsigned char* wring = stages_base + size_t(p.stages) * p.stage_bytes;     // [4 pairs][SP_WRING][32 rows x 128 B], swizzled
  unsigned char* eps_s = wring + 4 * SP_WRING * 4096;                         // [eps_rows][e_pitch]
  uint64_t* full = reinterpret_cast<uint64_t*>(eps_s + size_t(p.eps_rows) * p.e_pitch);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;     // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint64_t* wd_ready = acc_empty + 2;
  uint64_t* wd_free = wd_ready + 1;
  uint64_t* tbl_ready = wd_free + 1;
  uint64_t* pair_ready = tbl_ready + 1;      // [8] per epilogue warp: the partner's values are in its buffer
  uint64_t* pair_done = pair_ready + 8;      // [8] ... and it has finished with them
  uint64_t* wfree = pair_done + 8;           // [4 pairs][SP_WRING] both warps of the pair have read the W tile
  uint64_t* wfull = wfree + 4 * SP_WRING;    // [4 pairs][SP_WRING] a W tile has landed
  uint64_t* eps_full = wfull + 4 * SP_WRING; // the noise rows have landed (once)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(eps_full + 1);
  const int table_maps_bytes = ((2 * (p.Cout + p.Cin)) + 15) & ~15;
  const int table_bytes = table_maps_bytes + 4 * p.Cout;
  unsigned char* tables = reinterpret_cast<unsigned char*>(tmem_slot) + 16;
  float* xchg = reinterpret_cast<float*>(tables + 2 * size_t(table_bytes));      // [8 warps][32][17]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ksz = p.kh * p.kw;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    mbar_init(wd_ready, 8);
    mbar_init(wd_free, 1);
    mbar_init(tbl_ready, 8);
    for (int i = 0; i < 8; ++i) { mbar_init(&pair_ready[i], 1); mbar_init(&pair_done[i], 1); }
    for (int i = 0; i < 4 * SP_WRING; ++i) { mbar_init(&wfull[i], 1); mbar_init(&wfree[i], 2); }
    mbar_init(eps_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512u);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ producer: the noise rows once, then the hi run
      // and the lo run of every tile
      if (p.eps_rows > 0) {
        const uint32_t row_bytes = uint32_t(ksz) * 256u;
        mbar_expect_tx(eps_full, uint32_t(p.eps_rows) * row_bytes);
        for (int r = 0; r < p.eps_rows; ++r)
          bulk_load_1d(eps_s + size_t(r) * p.e_pitch, p.noise_t + size_t(r) * ksz * 64, row_bytes, eps_full);
      }
      uint32_t g = 0, tt = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        const long long d = u / p.sign_groups;
        long long r0, r1; float s;
        bf_unit_range(p, u % p.sign_groups, r0, r1, s);
        for (long long r = r0; r < r1 && ok; ++r) {
          const long long b = r * p.D + d;
          for (int ti = 0; ti < p.tiles_img && ok; ++ti, ++tt) {
            const long long row0 = b * (long long)p.img_rows + (long long)ti * NT;
            for (int half = 0; half < 2; ++half, ++g) {
              const int st = g % p.stages;
              const uint32_t phs = (g / p.stages) & 1;
              if (!mbar_wait(&empty[st], phs ^ 1, 1)) { ok = false; break; }
              CONV_TRACE(true, tt, half);
              mbar_expect_tx(&full[st], uint32_t(p.load_bytes));
              bulk_load_1d(stages_base + size_t(st) * p.stage_bytes, xs + (half ? p.lo_offset : 0) + row0 * 64, uint32_t(p.load_bytes), &full[st]);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer: the whole warp runs this loop in
    // converged control flow and one elected lane issues each instruction
    const uint32_t idesc = idesc_bf16(128, NT);
    const uint64_t desc0 = smem_desc_sw128(0);
    const uint32_t a_col0 = tmem_base + uint32_t(SP_A_COL);
    // pixel-row shift of every tap in 16-byte units (8 per 128-byte row), kept in registers: the issue loop below is
    // straight-line code, so that the instructions between two MMAs do not outlast the MMA itself (48 cycles)
    uint32_t xoff[9];
#pragma unroll
    for (int tap = 0; tap < 9; ++tap) {
      const int i = tap / p.kw, j = tap - i * p.kw;
      xoff[tap] = uint32_t(i * p.dh * p.Wp + j * p.dw) * 8u;
    }
    uint32_t g = 0, t = 0, ul = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      long long r0, r1; float s;
      bf_unit_range(p, u % p.sign_groups, r0, r1, s);
      if (r1 <= r0) continue;
      if (!warp_mbar_wait(wd_ready, ul & 1, 2)) { ok = false; break; }
      tc_fence_after();
      const long long ntiles = (r1 - r0) * p.tiles_img;
      for (long long ti = 0; ti < ntiles && ok; ++ti, ++t) {
        const uint32_t buf = t & 1;
        if (!warp_mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, 2)) { ok = false; break; }
        tc_fence_after();
        CONV_TRACE(lane == 0, t, 2);
        const uint32_t tmem_d = tmem_base + buf * uint32_t(NT);
        for (int half = 0; half < 2; ++half, ++g) {
          const int st = g % p.stages;
          const uint32_t phs = (g / p.stages) & 1;
          if (!warp_mbar_wait(&full[st], phs, 2)) { ok = false; break; }
          CONV_TRACE(lane == 0, t, 3 + 2 * half);
          const uint64_t x_desc = desc0 + uint64_t(smem_u32(stages_base + size_t(st) * p.stage_bytes) >> 4);
#pragma unroll
          for (int tap = 0; tap < 9; ++tap) {
            if (tap < ksz) {
              // 4 K steps of 8 tensor-memory columns per tap; only the tile's very first MMA overwrites the accumulator
#pragma unroll
              for (int k = 0; k < 4; ++k)
                warp_mma_bf16_tmem_a(tmem_d, a_col0 + uint32_t(tap * 32 + 8 * k), x_desc + uint64_t(xoff[tap] + 2 * k), idesc,
                                     (tap == 0 && k == 0) ? uint32_t(half) : 1u);
            }
          }
          warp_mma_commit(&empty[st]);
          CONV_TRACE(lane == 0, t, 4 + 2 * half);
        }
        warp_mma_commit(&acc_full[buf]);
      }
      warp_mma_commit(wd_free);
      ++ul;
    }
  } else {
    // ---------------------------------------------------------------------- filter builders / epilogue
    const int bt = threadIdx.x - 64;            // builder thread 0..255
    const int q = warp & 3;                     // tensor-memory lane quadrant of this warp
    const int hsel = (warp - 2) >> 2;           // which of the quadrant's two warps
    const int frow = q * 32 + lane;             // filter row = tensor-memory lane
    const bool lo_part = frow >= 64;
    const uint32_t lane_base = tmem_base + (uint32_t(q * 32) << 16);
    const int HoWo = p.Ho * p.Wo;
    // epilogue roles
    const bool upper = q >= 2;
    const int chan0 = (q & 1) * 32;
    const int mine = warp - 2, theirs = upper ? mine + 2 : mine - 2;
    float* my_buf = xchg + size_t(mine) * 32 * 17;
    float* their_buf = xchg + size_t(theirs) * 32 * 17;
    const int col_lo = hsel * (NT / 2);
    const int pos = lane & 15, rsel = lane >> 4;
    // filter build: the pair's ring of W tiles and its barriers; every member takes the same ksz groups in the same
    // order, so the tiles are a fixed cyclic sequence and can be requested across member boundaries
    const int pair = (q & 1) + 2 * hsel;
    unsigned char* wtiles = wring + size_t(pair) * SP_WRING * 4096;
    uint64_t* wbar = wfull + pair * SP_WRING;
    uint64_t* wdone = wfree + pair * SP_WRING;
    uint32_t my_groups = 0;                     // groups this pair consumes in the whole kernel (32-bit: cheap % and /)
    for (int u = blockIdx.x; u < p.units; u += gridDim.x) {
      long long r0, r1; float s;
      bf_unit_range(p, u % p.sign_groups, r0, r1, s);
      if (r1 > r0) my_groups += uint32_t(ksz);
    }
    auto request_w = [&](uint32_t nseq) {      // one lane of the pair: group number nseq of the pair's sequence
      const int G = hsel * ksz + int(nseq % uint32_t(ksz));
      const int slot = int(nseq % uint32_t(SP_WRING));
      mbar_expect_tx(&wbar[slot], 4096u);
      tma_load_2d(wtiles + size_t(slot) * 4096, &map_w, &wbar[slot], (G >> 1) * 64 + (G & 1) * 32, chan0);
    };
    if (!upper && lane == 0)
      for (uint32_t i = 0; i < uint32_t(SP_WRING) && i < my_groups; ++i) request_w(i);
    uint32_t n_w = 0;                           // groups consumed so far
    uint32_t t = 0, ul = 0, n_give = 0, n_take = 0;
    bool ok = true;
    if (p.eps_rows > 0 && !mbar_wait_relaxed(eps_full, 0, 4)) ok = false;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      const long long d = u / p.sign_groups;
      long long r0, r1; float s;
      bf_unit_range(p, u % p.sign_groups, r0, r1, s);
      if (r1 <= r0) continue;
      unsigned char* tb = tables + size_t(ul & 1) * table_bytes;
      int16_t* omap_s = reinterpret_cast<int16_t*>(tb);
      int16_t* imap_s = omap_s + p.Cout;
      float* add_s = reinterpret_cast<float*>(tb + table_maps_bytes);
      for (int c = bt; c < p.Cout; c += 256) {
        omap_s[c] = p.omap[d * p.Cout + c];
        float a = p.bias ? __ldg(p.bias + c) : 0.f;
        if (p.bias_noise) a += s * __ldg(p.bias_noise + d * p.Cout + c);
        add_s[c] = a;
      }
      for (int c = bt; c < p.Cin; c += 256) imap_s[c] = p.imap[d * p.Cin + c];
      __syncwarp();
      if (lane == 0) mbar_arrive(tbl_ready);
      if (!mbar_wait_relaxed(tbl_ready, ul & 1, 4)) { ok = false; break; }
      if (!mbar_wait_relaxed(wd_free, (ul & 1) ^ 1, 4)) { ok = false; break; }
      tc_fence_after();
      CONV_TRACE(threadIdx.x == 128, t, 9);
      {
        // 2 * ksz groups of (tap, 32 channels) = 16 tensor-memory columns each, ksz of them per warp pair.  This
        // thread's row: W from the tile (16-byte chunk z of row r sits at chunk z ^ (r & 7)), eps from the resident rows
        const bool has_row = chan0 + lane < p.Cout;
        const int so = (has_row && p.eps_rows > 0) ? int(omap_s[chan0 + lane]) : -1;
        // A tile is requested again (for the group SP_WRING further on) once both warps have read it.  The two warps
        // take turns with the requests, and each request is made one group late, when the partner has long arrived:
        // the warps never wait for each other here, and the few hundred ns a request costs its issuer are spread.
        auto rerequest = [&](uint32_t m) -> bool {
          if (upper != ((m & 1u) != 0) || m + SP_WRING >= my_groups) return true;
          const bool done = mbar_wait(&wdone[m % SP_WRING], (m / SP_WRING) & 1u, 4);
          if (__all_sync(0xffffffffu, done ? 1 : 0) == 0) return false;
          if (lane == 0) request_w(m + SP_WRING);
          return true;
        };
        int pending = -1;
#pragma unroll 1
        for (int gi = 0; gi < ksz; ++gi, ++n_w) {
          const int G = hsel * ksz + gi;
          const int tap = G >> 1, c0 = (G & 1) * 32;
          const int slot = int(n_w % SP_WRING);
          if (!mbar_wait(&wbar[slot], (n_w / SP_WRING) & 1u, 4)) { ok = false; break; }
          CONV_TRACE(threadIdx.x == 128 && ul == 1, 40 + gi, 11);
          const unsigned char* wrow = wtiles + size_t(slot) * 4096 + lane * 128;
          const unsigned char* erow = eps_s + size_t(so < 0 ? 0 : so) * p.e_pitch + tap * 256 + c0 * 4;
          uint32_t w16[16];
#pragma unroll
          for (int z = 0; z < 8; ++z) {
            const float4 w = *reinterpret_cast<const float4*>(wrow + ((z ^ (lane & 7)) << 4));
            float4 e = make_float4(0.f, 0.f, 0.f, 0.f);
            if (so >= 0) e = *reinterpret_cast<const float4*>(erow + 16 * z);
            const float f0 = fmaf(s, e.x, w.x), f1 = fmaf(s, e.y, w.y), f2 = fmaf(s, e.z, w.z), f3 = fmaf(s, e.w, w.w);
            // hi = the two values rounded to bf16 (one packed conversion); lo = what that rounding left over
            uint32_t p01 = pack_bf16(f0, f1), p23 = pack_bf16(f2, f3);
            if (lo_part) {
              p01 = pack_bf16(f0 - __uint_as_float(p01 << 16), f1 - __uint_as_float(p01 & 0xffff0000u));
              p23 = pack_bf16(f2 - __uint_as_float(p23 << 16), f3 - __uint_as_float(p23 & 0xffff0000u));
            }
            w16[2 * z] = p01;
            w16[2 * z + 1] = p23;
          }
          tmem_st16(lane_base + uint32_t(SP_A_COL + G * 16), w16);
          CONV_TRACE(threadIdx.x == 128 && ul == 1, 40 + gi, 12);
          __syncwarp();
          if (lane == 0) mbar_arrive(&wdone[slot]);             // this warp has read the tile
          if (pending >= 0 && !rerequest(uint32_t(pending))) { ok = false; break; }
          pending = int(n_w);
          CONV_TRACE(threadIdx.x == 128 && ul == 1, 40 + gi, 13);
        }
        if (ok && pending >= 0 && !rerequest(uint32_t(pending))) ok = false;
        tmem_st_wait();
        if (!ok) break;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(wd_ready);
      CONV_TRACE(threadIdx.x == 128, t, 10);

      const float add = (chan0 + lane < p.Cout) ? add_s[chan0 + lane] : 0.f;
      for (long long r = r0; r < r1 && ok; ++r) {
        const long long b = r * p.D + d;
        float* img = p.y + size_t(b) * p.Cout * HoWo;
        for (int ti = 0; ti < p.tiles_img && ok; ++ti, ++t) {
          const uint32_t buf = t & 1;
          if (!mbar_wait_relaxed(&acc_full[buf], (t >> 1) & 1, 3)) { ok = false; break; }
          tc_fence_after();
          CONV_TRACE(threadIdx.x == 128, t, 7);
          const bool live = (timeouts_so_far() == timeouts_at_start);
          const uint32_t tcol = lane_base + buf * uint32_t(NT) + uint32_t(col_lo);
          // chunk 0 is finished by the lower-row warp, chunk 1 by the upper-row warp, chunk 2 by one of them in turn
          const bool takes_third = (upper == ((t & 1) != 0));
          uint32_t c_own[16], c_other[16], c_third[16];
          tmem_ld16_nowait(tcol + (upper ? 16u : 0u), c_own);
          tmem_ld16_nowait(tcol + (upper ? 0u : 16u), c_other);
          tmem_ld16_nowait(tcol + 32u, c_third);
          tmem_ld_wait();
#pragma unroll
          for (int step = 0; step < 3 && ok; ++step) {
            // step 0: hand chunk `other` over; step 1: finish chunk `own`; step 2: the third chunk, either way
            const bool give = (step == 0) || (step == 2 && !takes_third);
            const uint32_t* src = (step == 0) ? c_other : (step == 1 ? c_own : c_third);
            if (give) {
              if (n_give > 0 && !mbar_wait(&pair_done[theirs], (n_give - 1) & 1, 3)) { ok = false; break; }
#pragma unroll
              for (int j = 0; j < 16; ++j) their_buf[lane * 17 + j] = __uint_as_float(src[j]);
              __syncwarp();
              if (lane == 0) mbar_arrive(&pair_ready[theirs]);
              ++n_give;
            } else {
              if (!mbar_wait(&pair_ready[mine], n_take & 1, 3)) { ok = false; break; }
              float v[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(src[j]) + my_buf[lane * 17 + j] + add;
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 16; ++j) my_buf[lane * 17 + j] = v[j];
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = my_buf[(2 * i + rsel) * 17 + pos];
              const int chunk = (step == 1) ? (upper ? 1 : 0) : 2;
              const int qpos = ti * NT + col_lo + chunk * 16 + pos;
              const int oy = qpos / p.Wp, ox = qpos - oy * p.Wp;
              if (live && oy < p.Ho && ox < p.Wo) {
                float* dst = img + size_t(chan0 + rsel) * HoWo + oy * p.Wo + ox;
#pragma unroll
                for (int i = 0; i < 16; ++i)
                  if (chan0 + 2 * i + rsel < p.Cout) dst[size_t(2 * i) * HoWo] = v[i];
              }
              __syncwarp();
              if (lane == 0) mbar_arrive(&pair_done[mine]);
              ++n_take;
            }
          }
          tc_fence_before();
          __syncwarp();
          CONV_TRACE(threadIdx.x == 128, t, 8);
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
    tmem_dealloc(tmem_base, 512u);
  }
}

// x (B,C,H,W) fp32 -> staged bf16 layout: for every image and 64-channel chunk a run of img_rows pixel rows
// (zero-padded image, pitch Wp, 128 bytes = 64 bf16 channels per row), 16-byte groups permuted by (row mod 8)
// as the 128-byte shared-memory swizzle does.  With SPLIT the lo copy (the bf16 rounding of what the hi copy left
// over) is written `lo_units` 16-byte units behind the hi copy, in the same layout.
//
// A streaming pass without block-wide synchronisation: one warp per (image, chunk, padded image row, run of 32
// pixels).  A lane reads its pixel from the 64 channel planes (64 coalesced 128-byte loads per warp, all in flight
// together), converts, and writes its 128-byte row into the warp's shared-memory tile; the warp then reads the tile
// back so that eight consecutive lanes hold one row and stores four whole rows (512 contiguous bytes) per instruction.
constexpr int STAGE_WARPS = 8;

template <bool SPLIT>
__global__ void __launch_bounds__(STAGE_WARPS * 32) stage_rows_bf16_kernel(const float* __restrict__ x, uint4* __restrict__ out,
                                                                         int C, int H, int W, int Hp, int Wp, int ph, int pw,
                                                                         int cchunks, int img_rows, long long lo_units,
                                                                         int runs, long long jobs) {
  __shared__ uint4 tiles[STAGE_WARPS][32 * 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint4* tile = tiles[warp];
  const long long nwarps = (long long)gridDim.x * STAGE_WARPS;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const size_t plane = size_t(H) * W;
  for (long long job = (long long)blockIdx.x * STAGE_WARPS + warp; job < jobs; job += nwarps) {
    const int xr = int(job % runs);
    const long long jr = job / runs;
    const int yp = int(jr % Hp);
    const long long bc = jr / Hp;                       // image * cchunks + chunk
    const int cc = int(bc % cchunks);
    const long long b = bc / cchunks;
    uint4* drow = out + (size_t(bc) * img_rows + size_t(yp) * Wp) * 8;      // eight 16-byte units per staged row
    const int yy = yp - ph;
    if (yy < 0 || yy >= H) {
      if (xr == 0)
        for (int i = lane; i < Wp * 8; i += 32) {
          drow[i] = zero;
          if (SPLIT) drow[i + lo_units] = zero;
        }
      continue;
    }
    if (xr == 0)
      for (int i = lane; i < pw * 8; i += 32) {            // the padding pixels left and right of the row
        drow[i] = zero;
        drow[size_t(pw + W) * 8 + i] = zero;
        if (SPLIT) { drow[i + lo_units] = zero; drow[size_t(pw + W) * 8 + i + lo_units] = zero; }
      }
    const int x0 = xr * 32;
    const int xx = x0 + lane;
    const bool valid = xx < W;
    const float* src = x + ((size_t(b) * C + size_t(cc) * 64) * H + yy) * W + xx;
    float v[64];
#pragma unroll
    for (int c = 0; c < 64; ++c) v[c] = valid ? __ldcs(src + size_t(c) * plane) : 0.f;
    const int row0 = yp * Wp + pw + x0;                // staged row of the run's first pixel (img_rows is a multiple of 8)
    uint4* d0 = drow + size_t(pw + x0) * 8;
#pragma unroll
    for (int part = 0; part < (SPLIT ? 2 : 1); ++part) {
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        uint32_t w[4];
#pragma unroll
        for (int z = 0; z < 4; ++z) {
          const float a = v[8 * g + 2 * z], bb = v[8 * g + 2 * z + 1];
          uint32_t pk = pack_bf16(a, bb);
          if (part == 1) pk = pack_bf16(a - __uint_as_float(pk << 16), bb - __uint_as_float(pk & 0xffff0000u));
          w[z] = pk;
        }
        tile[lane * 8 + (g ^ (lane & 7))] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      __syncwarp();
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int r = (lane >> 3) + 4 * it;            // pixel of the run; eight lanes per row
        const int pos = lane & 7;                      // 16-byte position in the staged row
        const int chunk = pos ^ ((row0 + r) & 7);      // the channel group that belongs there
        const uint4 val = tile[r * 8 + (chunk ^ (r & 7))];
        if (x0 + r < W) d0[size_t(r) * 8 + pos + (part ? lo_units : 0)] = val;
      }
      __syncwarp();
    }
  }
}

__global__ void reorder_filter_bf_kernel(const float* __restrict__ src, float* __restrict__ dst, int N, int C, int ksz) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= N * C * ksz) return;
  const int n = idx / (C * ksz);
  const int rem = idx - n * C * ksz;
  const int tap = rem / C, c = rem - tap * C;
  dst[idx] = src[(size_t(n) * C + c) * ksz + tap];
}

int conv_bf16_error_word(int* v, bool clear) { return read_error_word(v, clear, "tc_error_flag"); }

static int64_t bf_align256(int64_t v) { return (v + 255) & ~int64_t(255); }

struct ConvBfPlan { ConvBfParams p; size_t smem; int64_t x_bytes, map_bytes, filt_bytes; };

// form 0: filter in shared memory (conv_bf16_kernel); form 1: three-term form with the filter in tensor memory
// form 1 additionally needs identity input channels (no input permutation, in_sp == Cin) and the noise rows to fit in
// shared memory beside the pipeline (80 KB at most: 32 rows of a 3x3 filter)
static bool tmem_form_covers(int Cin, int Cout, int kh, int kw, int eps_rows) {
  return Cin == 64 && Cout <= 64 && kh * kw <= 9 && eps_rows >= 0 && size_t(eps_rows) * (size_t(kh) * kw * 256 + 16) <= 80 * 1024;
}

static int plan_conv_bf16(ConvBfPlan& pl, int64_t D, int64_t R, int Cin, int H, int W, int Cout, int kh, int kw,
                          int sh, int sw, int ph, int pw, int dh, int dw, int antithetic, const char* what, int terms = 1,
                          int form = 0, int eps_rows = 0) {
  NES_REQUIRE(form == 0 || (terms == 3 && tmem_form_covers(Cin, Cout, kh, kw, eps_rows)), NES_ERR_UNSUPPORTED,
              "%s: the tensor-memory filter form needs Cin = 64, Cout <= 64, at most 9 taps and at most 80 KB of noise rows", what);
  const int NT = form == 1 ? SP_NT : (terms == 3 ? BF_NT3 : BF_NT);
  NES_REQUIRE(D >= 0 && R >= 0 && Cin > 0 && H > 0 && W > 0 && Cout > 0 && kh > 0 && kw > 0 && ph >= 0 && pw >= 0 &&
              dh > 0 && dw > 0, NES_ERR_BAD_ARG, "%s: bad geometry", what);
  NES_REQUIRE(sh == 1 && sw == 1, NES_ERR_UNSUPPORTED, "%s: the bf16 tensor-core path needs stride 1", what);
  NES_REQUIRE(Cin % 64 == 0, NES_ERR_UNSUPPORTED, "%s: the bf16 tensor-core path needs Cin %% 64 == 0 (got %d)", what, Cin);
  NES_REQUIRE(Cout % 8 == 0 && Cout <= 128, NES_ERR_UNSUPPORTED, "%s: the bf16 tensor-core path needs Cout %% 8 == 0 and <= 128 (got %d)", what, Cout);
  ConvBfParams& p = pl.p;
  p.Cin = Cin; p.H = H; p.W = W; p.Cout = Cout; p.kh = kh; p.kw = kw; p.ph = ph; p.pw = pw; p.dh = dh; p.dw = dw;
  p.Ho = H + 2 * ph - dh * (kh - 1);
  p.Wo = W + 2 * pw - dw * (kw - 1);
  NES_REQUIRE(p.Ho > 0 && p.Wo > 0, NES_ERR_BAD_ARG, "%s: empty output", what);
  p.Hp = H + 2 * ph; p.Wp = W + 2 * pw;
  p.M = Cout <= 64 ? 64 : 128;
  p.tmem_filter = form;
  p.eps_rows = form == 1 ? eps_rows : 0;
  p.e_pitch = kh * kw * 256 + 16;                    // 16 bytes more than a row: rows start in different bank groups
  if (form == 1) p.M = 128;
  p.tiles_img = ceil_div(p.Ho * p.Wp, NT);
  const int max_shift = (kh - 1) * dh * p.Wp + (kw - 1) * dw;
  p.img_rows = (p.Hp * p.Wp + 7) & ~7;
  p.load_bytes = (NT + max_shift) * 128;
  p.stage_bytes = (p.load_bytes + 1023) & ~1023;
  p.D = D; p.R = R; p.antithetic = antithetic;
  p.sign_groups = antithetic ? 2 : 1;
  NES_REQUIRE(D * p.sign_groups <= INT32_MAX && D * R <= INT32_MAX, NES_ERR_UNSUPPORTED, "%s: population too large", what);
  p.units = int(D * p.sign_groups);
  p.cchunks = Cin / 64;
  p.kchunks = kh * kw * p.cchunks;
  const size_t wd_bytes = form == 1 ? 0 : size_t(terms == 3 ? 2 : 1) * p.kchunks * p.M * 128;
  const size_t table_bytes = (((2 * (size_t(Cout) + Cin)) + 15) & ~size_t(15)) + 4 * size_t(Cout);
  // form 1: the epilogue's exchange buffers [8 warps][32][17], the ring of W tiles [4 pairs][SP_WRING][4096 B] and the
  // resident noise rows
  const size_t xpose_bytes = form == 1 ? 8 * size_t(32) * 17 * sizeof(float) + 4 * size_t(SP_WRING) * 4096 + size_t(p.eps_rows) * p.e_pitch
                                       : 8 * size_t(p.M == 128 ? 32 : 16) * 33 * sizeof(float);
  const size_t fixed = 1024 + wd_bytes + 400 + 16 + 16 + 2 * table_bytes + 8 * size_t(kh) * kw + xpose_bytes;
  const size_t limit = 227 * 1024;
  NES_REQUIRE(fixed + 2 * (size_t(p.stage_bytes) + 16) <= limit, NES_ERR_UNSUPPORTED,
              "%s: the member filter (%zu bytes) plus two input stages (%d bytes each) do not fit in shared memory on the "
              "bf16 tensor-core path", what, wd_bytes, p.stage_bytes);
  int stages = int((limit - fixed) / (size_t(p.stage_bytes) + 16));
  if (stages > 6) stages = 6;
  if (terms == 3 && stages > 4) stages = 4;
  if (form == 1) {                                  // hi / lo slot pairs, up to four tiles in flight
    stages = int((limit - fixed) / (size_t(p.stage_bytes) + 16)) & ~1;
    if (stages > 8) stages = 8;
  }
  p.stages = stages;
  pl.smem = 1024 + wd_bytes + size_t(stages) * p.stage_bytes + (2 * stages + 48) * sizeof(uint64_t) + 16 + 16 + 2 * table_bytes +
            8 * size_t(kh) * kw + xpose_bytes;
  const int64_t copy_bytes = bf_align256(D * R * int64_t(p.cchunks) * p.img_rows * 128 + int64_t(p.stage_bytes));
  p.lo_offset = copy_bytes / 2;                    // bf16 elements
  pl.x_bytes = (terms == 3 ? 2 : 1) * copy_bytes;
  pl.map_bytes = bf_align256(D * (int64_t(Cin) + Cout) * 2);
  pl.filt_bytes = bf_align256(int64_t(Cout) * Cin * kh * kw * 4);
  return NES_OK;
}

static int run_conv_bf16(ConvBfPlan& pl, const float* x, void* x_staged, cudaStream_t st, const char* what, int terms = 1) {
  ConvBfParams& p = pl.p;
  const int64_t B = p.D * p.R;
  const int runs = ceil_div(p.W, 32);
  const long long jobs = B * int64_t(p.cchunks) * p.Hp * runs;          // one warp per (image, chunk, padded row, 32 pixels)
  const long long lo_units = p.lo_offset / 8;                           // bf16 elements -> 16-byte units
  long long sblocks = (jobs + STAGE_WARPS - 1) / STAGE_WARPS;
  if (sblocks > 16LL * sm_count()) sblocks = 16LL * sm_count();
  if (sblocks < 1) sblocks = 1;
  uint4* xo = static_cast<uint4*>(x_staged);
  if (terms == 3) stage_rows_bf16_kernel<true><<<(unsigned)sblocks, STAGE_WARPS * 32, 0, st>>>(x, xo, p.Cin, p.H, p.W, p.Hp, p.Wp, p.ph, p.pw, p.cchunks, p.img_rows, lo_units, runs, jobs);
  else stage_rows_bf16_kernel<false><<<(unsigned)sblocks, STAGE_WARPS * 32, 0, st>>>(x, xo, p.Cin, p.H, p.W, p.Hp, p.Wp, p.ph, p.pw, p.cchunks, p.img_rows, 0, runs, jobs);
  int rc = check_launch(what);
  if (rc != NES_OK) return rc;
  int grid = p.units < sm_count() ? p.units : sm_count();
  if (grid < 1) grid = 1;
  if (p.tmem_filter) {
    // W re-ordered to (n, tap, c): a (Cout, K) fp32 matrix read in tiles of 32 rows x 32 channels, 128-byte swizzle
    EncodeTiledFn fn = encode_fn();
    NES_REQUIRE(fn != nullptr, NES_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", what);
    CUtensorMap map_w;
    const cuuint64_t K = cuuint64_t(p.kh) * p.kw * 64;
    cuuint64_t dims[2] = {K, (cuuint64_t)p.Cout};
    cuuint64_t strides[1] = {K * sizeof(float)};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&map_w, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(p.weight_t), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    NES_REQUIRE(r == CUDA_SUCCESS, NES_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
    cudaError_t e = cudaFuncSetAttribute(conv_split_tmem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
    if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "%s: shared memory opt-in failed: %s", what, cudaGetErrorString(e));
    conv_split_tmem_kernel<<<grid, BF_THREADS, pl.smem, st>>>(map_w, static_cast<const __nv_bfloat16*>(x_staged), p);
    return check_launch(what);
  }
  auto kern = terms == 3 ? conv_bf16_kernel<3, BF_NT3> : conv_bf16_kernel<1, BF_NT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "%s: shared memory opt-in failed: %s", what, cudaGetErrorString(e));
  kern<<<grid, BF_THREADS, pl.smem, st>>>(static_cast<const __nv_bfloat16*>(x_staged), p);
  return check_launch(what);
}

}  // namespace tc
}  // namespace nes

#ifdef NES_CONV_TRACE
// instrumented builds only: copies the 64 x 16 timeline slots of block 0 to host memory
extern "C" int nes_debug_conv_trace(long long* out) {
  return cudaMemcpyFromSymbol(out, nes::tc::g_conv_trace, sizeof(long long) * 64 * 16) == cudaSuccess ? 0 : 1;
}
#endif

using namespace nes;
using namespace nes::tc;

static int64_t bf16_scratch_bytes(int64_t D, int64_t R, int Cin, int H, int W, int Cout, int kh, int kw, int ph, int pw, int copies) {
  if (D <= 0 || R <= 0) return 0;
  const int64_t hp = H + 2 * ph, wp = W + 2 * pw;
  const int64_t img_rows = (hp * wp + 7) & ~int64_t(7);
  const int64_t tail = ((BF_NT + (kh - 1) * wp * 8 + (kw - 1) * 8) * 128 + 1023) & ~int64_t(1023);   // covers any dilation <= 8
  return copies * bf_align256(D * R * int64_t((Cin + 63) / 64) * img_rows * 128 + tail) + bf_align256(D * (int64_t(Cin) + Cout) * 2) +
         2 * bf_align256(int64_t(Cout) * Cin * kh * kw * 4);
}

extern "C" int64_t nes_conv2d_fwd_bf16_scratch_bytes(int64_t D, int64_t R, int Cin, int H, int W, int Cout, int kh, int kw,
                                                     int ph, int pw) {
  return bf16_scratch_bytes(D, R, Cin, H, W, Cout, kh, kw, ph, pw, 1);
}

extern "C" int64_t nes_conv2d_fwd_bf16x3_scratch_bytes(int64_t D, int64_t R, int Cin, int H, int W, int Cout, int kh, int kw,
                                                       int ph, int pw) {
  return bf16_scratch_bytes(D, R, Cin, H, W, Cout, kh, kw, ph, pw, 2);
}

// 1 when the split-bf16 tensor-core form covers the geometry (stride 1, Cin a multiple of 64, Cout a multiple of 8 up
// to 128, both filter copies plus two input slots within shared memory), else 0
extern "C" int nes_conv2d_fwd_bf16x3_supported(int Cin, int H, int W, int Cout, int kh, int kw, int sh, int sw,
                                               int ph, int pw, int dh, int dw) {
  ConvBfPlan pl;
  if (Cin <= 0 || H <= 0 || W <= 0 || Cout <= 0 || kh <= 0 || kw <= 0 || ph < 0 || pw < 0 || dh <= 0 || dw <= 0) return 0;
  if (dh > 8 || dw > 8) return 0;
  return plan_conv_bf16(pl, 1, 1, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, 0, "conv2d_fwd_bf16x3", 3) == NES_OK ? 1 : 0;
}

// The same question for a permuted-noise layer: output-permuted layers with 64 input channels may also take the form
// with the filter in tensor memory, which needs far less shared memory (larger images fit).
extern "C" int nes_permuted_conv2d_fwd_bf16x3_supported(int Cin, int H, int W, int Cout, int kh, int kw, int sh, int sw,
                                                        int ph, int pw, int dh, int dw, int in_sp, int out_sp,
                                                        int input_permutations) {
  if (nes_conv2d_fwd_bf16x3_supported(Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw)) return 1;
  if (Cin <= 0 || H <= 0 || W <= 0 || Cout <= 0 || kh <= 0 || kw <= 0 || ph < 0 || pw < 0 || dh <= 0 || dw <= 0) return 0;
  if (dh > 8 || dw > 8 || input_permutations || in_sp != Cin || !tmem_form_covers(Cin, Cout, kh, kw, out_sp)) return 0;
  ConvBfPlan pl;
  return plan_conv_bf16(pl, 1, 1, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, 0, "permuted_conv2d_fwd_bf16x3", 3, 1, out_sp) == NES_OK
             ? 1 : 0;
}

static int perturbed_conv_bf16(int terms, const float* x, const float* weight, const float* bias,
                               const float* noise, const float* bias_noise, float* y,
                               int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                               int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                               int antithetic, void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  ConvBfPlan pl;
  int rc = plan_conv_bf16(pl, D, R, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, antithetic, "perturbed_conv2d_fwd_bf16", terms);
  if (rc != NES_OK) return rc;
  if (D == 0 || R == 0) return NES_OK;
  NES_REQUIRE(x && weight && noise && y, NES_ERR_BAD_ARG, "perturbed_conv2d_fwd_bf16: null pointer");
  NES_REQUIRE(scratch && scratch_bytes >= pl.x_bytes && (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, NES_ERR_SCRATCH,
              "perturbed_conv2d_fwd_bf16: scratch needs %lld bytes, 256-byte aligned", (long long)pl.x_bytes);
  pl.p.weight = weight; pl.p.bias = bias; pl.p.bias_noise = bias_noise; pl.p.y = y;
  pl.p.noise_kind = 1; pl.p.noise = noise; pl.p.omap = nullptr; pl.p.imap = nullptr; pl.p.in_sp = Cin;
  pl.p.weight_t = nullptr; pl.p.noise_t = nullptr; pl.p.identity_in = 1;
  pl.p.dense_vec = (aligned16(weight) && aligned16(noise)) ? 1 : 0;
  return run_conv_bf16(pl, x, scratch, as_stream(stream), "perturbed_conv2d_fwd_bf16", terms);
}

extern "C" int nes_perturbed_conv2d_fwd_bf16(const float* x, const float* weight, const float* bias,
                                             const float* noise, const float* bias_noise, float* y,
                                             int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                             int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                             int antithetic, void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  return perturbed_conv_bf16(1, x, weight, bias, noise, bias_noise, y, D, R, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw,
                             antithetic, scratch, scratch_bytes, stream);
}

extern "C" int nes_perturbed_conv2d_fwd_bf16x3(const float* x, const float* weight, const float* bias,
                                               const float* noise, const float* bias_noise, float* y,
                                               int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                               int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                               int antithetic, void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  return perturbed_conv_bf16(3, x, weight, bias, noise, bias_noise, y, D, R, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw,
                             antithetic, scratch, scratch_bytes, stream);
}

static int permuted_conv_bf16(int terms, const float* x, const float* weight, const float* bias,
                              const float* eps, const float* bias_noise,
                              const int16_t* pin, const int16_t* pout, float* y,
                              int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                              int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                              int in_sp, int out_sp, int antithetic,
                              void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  ConvBfPlan pl;
  // the three-term form keeps the filter in tensor memory where that form covers the layer
  int form = (terms == 3 && sh == 1 && sw == 1 && pin == nullptr && in_sp == Cin &&
              tmem_form_covers(Cin, Cout, kh, kw, out_sp)) ? 1 : 0;
  int rc = plan_conv_bf16(pl, D, R, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, antithetic, "permuted_conv2d_fwd_bf16", terms, form,
                          out_sp);
  if (rc == NES_ERR_UNSUPPORTED && form == 1) {           // the other form may still fit
    form = 0;
    rc = plan_conv_bf16(pl, D, R, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, antithetic, "permuted_conv2d_fwd_bf16", terms, 0, 0);
  }
  if (rc != NES_OK) return rc;
  if (D == 0 || R == 0) return NES_OK;
  NES_REQUIRE(x && weight && eps && y, NES_ERR_BAD_ARG, "permuted_conv2d_fwd_bf16: null pointer");
  NES_REQUIRE(out_sp >= 0 && out_sp <= Cout && in_sp >= 0 && in_sp <= Cin && (pin || in_sp == Cin), NES_ERR_BAD_ARG,
              "permuted_conv2d_fwd_bf16: sparsity exceeds degree");
  NES_REQUIRE(pin || in_sp % 8 == 0, NES_ERR_UNSUPPORTED, "permuted_conv2d_fwd_bf16: in_sp must be a multiple of 8");
  const int64_t need = pl.x_bytes + pl.map_bytes + 2 * pl.filt_bytes;
  NES_REQUIRE(scratch && scratch_bytes >= need && (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0,
              NES_ERR_SCRATCH, "permuted_conv2d_fwd_bf16: scratch needs %lld bytes, 256-byte aligned", (long long)need);
  cudaStream_t st = as_stream(stream);
  unsigned char* sp = static_cast<unsigned char*>(scratch);
  int16_t* omap = reinterpret_cast<int16_t*>(sp + pl.x_bytes);
  int16_t* imap = omap + D * Cout;
  float* weight_t = reinterpret_cast<float*>(sp + pl.x_bytes + pl.map_bytes);
  float* eps_t = reinterpret_cast<float*>(sp + pl.x_bytes + pl.map_bytes + pl.filt_bytes);
  rc = launch_permuted_maps(pin, pout, omap, imap, D, Cin, Cout, in_sp, out_sp, st);
  if (rc != NES_OK) return rc;
  const int ksz = kh * kw;
  reorder_filter_bf_kernel<<<ceil_div(Cout * Cin * ksz, 256), 256, 0, st>>>(weight, weight_t, Cout, Cin, ksz);
  if ((rc = check_launch("permuted_conv2d_fwd_bf16(reorder W)")) != NES_OK) return rc;
  if (out_sp * in_sp > 0) {
    reorder_filter_bf_kernel<<<ceil_div(out_sp * in_sp * ksz, 256), 256, 0, st>>>(eps, eps_t, out_sp, in_sp, ksz);
    if ((rc = check_launch("permuted_conv2d_fwd_bf16(reorder eps)")) != NES_OK) return rc;
  }
  pl.p.weight = weight; pl.p.bias = bias; pl.p.bias_noise = bias_noise; pl.p.y = y;
  pl.p.noise_kind = 2; pl.p.noise = eps; pl.p.omap = omap; pl.p.imap = imap; pl.p.in_sp = in_sp;
  pl.p.weight_t = weight_t; pl.p.noise_t = eps_t; pl.p.identity_in = (pin == nullptr) ? 1 : 0;
  pl.p.dense_vec = 0;
  return run_conv_bf16(pl, x, scratch, st, "permuted_conv2d_fwd_bf16", terms);
}

extern "C" int nes_permuted_conv2d_fwd_bf16(const float* x, const float* weight, const float* bias,
                                            const float* eps, const float* bias_noise,
                                            const int16_t* pin, const int16_t* pout, float* y,
                                            int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                            int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                            int in_sp, int out_sp, int antithetic,
                                            void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  return permuted_conv_bf16(1, x, weight, bias, eps, bias_noise, pin, pout, y, D, R, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw,
                            dh, dw, in_sp, out_sp, antithetic, scratch, scratch_bytes, stream);
}

extern "C" int nes_permuted_conv2d_fwd_bf16x3(const float* x, const float* weight, const float* bias,
                                              const float* eps, const float* bias_noise,
                                              const int16_t* pin, const int16_t* pout, float* y,
                                              int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                              int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                              int in_sp, int out_sp, int antithetic,
                                              void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  return permuted_conv_bf16(3, x, weight, bias, eps, bias_noise, pin, pout, y, D, R, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw,
                            dh, dw, in_sp, out_sp, antithetic, scratch, scratch_bytes, stream);
}
