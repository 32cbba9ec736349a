// Tensor-core convolution for the per-member layers (PermutedConv2d / PerturbedConv2d), TF32 mode.
//
// The population forward is, per member d and antithetic sign s, an ordinary convolution with the
// member's effective filter W_d = W + s * E_d.  A persistent thread block takes (member, sign) units:
//   1. its four "builder" warps form W_d in shared memory -- from W and the shared noise through the
//      member's channel maps, or from the member's dense noise -- already rounded to TF32, reordered to
//      k = tap * Cin + c and laid out as the 128-byte-swizzled K-major tiles tcgen05.mma reads
//      (never materialised in HBM);
//   2. a producer thread streams the member's input out of a zero-padded channels-last copy of x viewed
//      as a 1-D sequence of pixels (pitch Wp = W + 2*pad): an output tile is 128 consecutive positions
//      q = y*Wp + x of that sequence, and filter tap (i,j) needs the same sequence shifted by
//      i*dil*Wp + j*dil.  So ONE staged run of 128 + max-shift pixels per (tile, 32-channel chunk) serves
//      all taps: the im2col expansion happens in shared memory, not in L2 traffic.  The copy is stored
//      chunk-major and already in the 128-byte-swizzled byte order of the shared-memory tile, so a run
//      is one contiguous range fetched by a single bulk async copy (cp.async.bulk + mbarrier);
//   3. one warp (converged, an elected lane) issues tcgen05.mma (kind::tf32, M = 128 positions, N = Cout, K = 8): per tap the A
//      descriptor simply starts (shift * 128 bytes) further into the same staged box (the box itself
//      starts on a 1024-byte boundary, so the swizzle pattern stays aligned and the descriptor's base
//      offset is 0); accumulators alternate between two tiles in tensor memory, so that
//   4. the builder warps, now epilogue warps, read the other accumulator with tcgen05.ld (one pixel per
//      thread), add bias + s * bias_noise and store NCHW rows while the next tile is multiplied.
// A pre-pass writes that padded, swizzled, TF32-rounded copy of x (the only extra HBM traffic).
// Positions that fall on padding columns (x >= Wo) are computed and dropped (2*pad/Wp of the work).
// All mbarrier waits are bounded (see tc_ptx.cuh); an error code is left in the device error word.
#include "tc_ptx.cuh"

namespace nes {

// defined in conv.cu
int launch_permuted_maps(const int16_t* pin, const int16_t* pout, int16_t* omap, int16_t* imap, int64_t D,
                         int Cin, int Cout, int in_sp, int out_sp, cudaStream_t st);

namespace tc {

constexpr int CONV_THREADS = 320;        // producer, MMA issuer, 4 epilogue + builder warps, 4 builder warps

struct ConvTcParams {
  int Cin, H, W, Cout, kh, kw, ph, pw, dh, dw, Ho, Wo;
  int Hp, Wp, tiles_img, img_rows, load_bytes, stage_bytes;
  long long D, R;
  int antithetic, sign_groups, units;
  int stages, kchunks, cchunks, tmem_cols;
  const float* weight; const float* bias; const float* bias_noise; float* y;
  int noise_kind;               // 0 none, 1 dense (D,Cout,Cin,ksz), 2 permuted (out_sp,in_sp,ksz) through omap / imap
  const float* noise; const int16_t* omap; const int16_t* imap; int in_sp;
  const float* weight_t; const float* noise_t;   // (n, tap, c) re-ordered copies for noise_kind 2
  int identity_in;                                // no input permutation: imap is the identity
};

// repeats [r0, r1) that belong to sign group sg, and the sign
__device__ __forceinline__ void unit_range(const ConvTcParams& p, int sg, long long& r0, long long& r1, float& s) {
  if (!p.antithetic) { r0 = 0; r1 = p.R; s = 1.f; return; }
  const long long half = (p.R + 1) / 2;
  if (sg == 0) { r0 = 0; r1 = half; s = 1.f; } else { r0 = half; r1 = p.R; s = -1.f; }
}

__global__ void __launch_bounds__(CONV_THREADS, 1) conv_tf32_kernel(const float* __restrict__ xs, const ConvTcParams p) {
  extern __shared__ unsigned char dyn_raw[];
  const unsigned int timeouts_at_start = timeouts_so_far();
  const uint32_t raw = smem_u32(dyn_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  unsigned char* wd = dyn_raw + pad;                                   // [kchunks][Cout][128 B]
  const int wd_chunk_bytes = p.Cout * 128;
  unsigned char* atiles = wd + size_t(p.kchunks) * wd_chunk_bytes;     // [stages][stage_bytes]: one staged pixel box each
  uint64_t* full = reinterpret_cast<uint64_t*>(atiles + size_t(p.stages) * p.stage_bytes);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;     // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint64_t* wd_ready = acc_empty + 2;
  uint64_t* wd_free = wd_ready + 1;
  uint64_t* tbl_ready = wd_free + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tbl_ready + 1);
  const int table_maps_bytes = ((2 * (p.Cout + p.Cin)) + 15) & ~15;
  const int table_bytes = table_maps_bytes + 4 * p.Cout;
  unsigned char* tables = reinterpret_cast<unsigned char*>(tmem_slot) + 16;    // two parities

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ksz = p.kh * p.kw;
  const int K = p.Cin * ksz;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    mbar_init(wd_ready, 8);
    mbar_init(wd_free, 1);
    mbar_init(tbl_ready, 8);
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
          const long long b = r * p.D + d;
          for (int ti = 0; ti < p.tiles_img && ok; ++ti) {
            for (int cc = 0; cc < p.cchunks; ++cc, ++g) {
              const int st = g % p.stages;
              const uint32_t phs = (g / p.stages) & 1;
              if (!mbar_wait(&empty[st], phs ^ 1, 1)) { ok = false; break; }
              const long long row0 = (b * p.cchunks + cc) * (long long)p.img_rows + (long long)ti * 128;
              mbar_expect_tx(&full[st], uint32_t(p.load_bytes));
              bulk_load_1d(atiles + size_t(st) * p.stage_bytes, xs + row0 * 32, uint32_t(p.load_bytes), &full[st]);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer: the whole warp runs this loop in
    // converged control flow and one elected lane issues each instruction (see warp_mma_tf32)
    // D = fp32, A = B = tf32, both K-major, M = 128 positions, N = output channels
    const uint32_t idesc = idesc_tf32(128, p.Cout);
    const uint64_t desc0 = smem_desc_sw128(0);
    const uint64_t wd_desc = desc0 + uint64_t(smem_u32(wd) >> 4);
    const uint32_t cc_step = uint32_t(wd_chunk_bytes >> 4);
    const uint32_t tap_step = uint32_t(p.cchunks) * cc_step;            // filter chunks of one tap
    uint32_t g = 0, t = 0, ul = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      long long r0, r1; float s;
      unit_range(p, u % p.sign_groups, r0, r1, s);
      if (r1 <= r0) continue;
      if (!warp_mbar_wait(wd_ready, ul & 1, 2)) { ok = false; break; }
      tc_fence_after();
      const long long ntiles = (r1 - r0) * p.tiles_img;
      for (long long ti = 0; ti < ntiles && ok; ++ti, ++t) {
        const uint32_t buf = t & 1;
        if (!warp_mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * uint32_t(p.Cout);
        for (int cc = 0; cc < p.cchunks; ++cc, ++g) {
          const int st = g % p.stages;
          const uint32_t phs = (g / p.stages) & 1;
          if (!warp_mbar_wait(&full[st], phs, 2)) { ok = false; break; }
          tc_fence_after();
          const uint64_t x_desc = desc0 + uint64_t(smem_u32(atiles + size_t(st) * p.stage_bytes) >> 4);
          const uint64_t w_desc = wd_desc + uint64_t(uint32_t(cc) * cc_step);
          uint32_t accumulate = (cc > 0) ? 1u : 0u;
          for (int i = 0, tap = 0; i < p.kh; ++i)
            for (int j = 0; j < p.kw; ++j, ++tap) {
              // pixel-row shift of the tap in 16-byte units (8 per 128-byte row); the tap's filter chunk
              const uint64_t al = x_desc + uint64_t(uint32_t(i * p.dh * p.Wp + j * p.dw) * 8u);
              const uint64_t bl = w_desc + uint64_t(uint32_t(tap) * tap_step);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                warp_mma_tf32(tmem_d, al + uint64_t(2 * k), bl + uint64_t(2 * k), idesc, accumulate);
                accumulate = 1u;
              }
            }
          warp_mma_commit(&empty[st]);
        }
        warp_mma_commit(&acc_full[buf]);
      }
      warp_mma_commit(wd_free);
      ++ul;
    }
  } else {
    // ---------------------------------------------------------------------- filter builders / epilogue
    // warps 2-5 build the member filter and then drain accumulators; warps 6-9 only build
    const int bt = threadIdx.x - 64;            // builder thread 0..255
    const bool drains = warp < 6;
    const int q = warp & 3;                     // TMEM lane quadrant an epilogue warp may read
    const int pix = q * 32 + lane;              // position of the tile = accumulator row
    const int HoWo = p.Ho * p.Wo;
    const int k4 = K / 4, c4n = p.Cin / 4;
    uint32_t t = 0, ul = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      const long long d = u / p.sign_groups;
      long long r0, r1; float s;
      unit_range(p, u % p.sign_groups, r0, r1, s);
      if (r1 <= r0) continue;
      // per-unit tables (double-buffered by unit parity): channel maps and bias + s * bias_noise
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
      if (lane == 0) mbar_arrive(tbl_ready);          // all eight builder warps have written their table entries
      if (!mbar_wait_relaxed(tbl_ready, ul & 1, 4)) { ok = false; break; }
      if (!mbar_wait_relaxed(wd_free, (ul & 1) ^ 1, 4)) { ok = false; break; }

      if (p.noise_kind == 1) {
        // dense member noise in its native (n, c, tap) order: coalesced reads, scattered 4-byte writes
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
            const int jc = kk >> 5, w32 = kk & 31;
            unsigned char* dst = wd + size_t(jc) * wd_chunk_bytes + (n >> 3) * 1024 + (n & 7) * 128 +
                                 ((((w32 >> 2) ^ (n & 7))) << 4) + (w32 & 3) * 4;
            *reinterpret_cast<float*>(dst) = round_tf32(fmaf(s, ev[i], wv[i]));
          }
        }
      } else {
        // W and eps were re-ordered to (n, tap, c): 128-bit reads along c, 128-bit swizzled writes
        const float4* Wt = reinterpret_cast<const float4*>(p.weight_t);
        const bool identity_in = p.identity_in != 0;
        const int groups = p.Cout * k4;
        // group index -> (n, rem) is carried incrementally (no division in the loop): +256 per step
        const int step_n = 256 / k4, step_r = 256 - step_n * k4;
        int n_cur = bt / k4, r_cur = bt - n_cur * k4;
        constexpr int BATCH = 6;
        for (int g0 = bt; g0 < groups; g0 += 256 * BATCH) {
          float4 wv[BATCH], ev[BATCH];
          int nn[BATCH], kk[BATCH];
#pragma unroll
          for (int i = 0; i < BATCH; ++i) {
            const int gidx = g0 + i * 256;
            wv[i] = make_float4(0.f, 0.f, 0.f, 0.f); ev[i] = wv[i]; nn[i] = -1; kk[i] = 0;
            if (gidx < groups) {
              const int n = n_cur, rem = r_cur;
              const int tap = rem / c4n, c = (rem - tap * c4n) * 4;
              nn[i] = n; kk[i] = tap * p.Cin + c;
              wv[i] = __ldg(Wt + gidx);
              const int so = (p.noise_kind == 2) ? int(omap_s[n]) : -1;
              if (so >= 0) {
                const float* er = p.noise_t + (size_t(so) * ksz + tap) * p.in_sp;
                if (identity_in) {
                  ev[i] = __ldg(reinterpret_cast<const float4*>(er + c));
                } else {
                  const int c0 = imap_s[c], c1 = imap_s[c + 1], c2 = imap_s[c + 2], c3 = imap_s[c + 3];
                  if (c0 >= 0) ev[i].x = __ldg(er + c0);
                  if (c1 >= 0) ev[i].y = __ldg(er + c1);
                  if (c2 >= 0) ev[i].z = __ldg(er + c2);
                  if (c3 >= 0) ev[i].w = __ldg(er + c3);
                }
              }
            }
            n_cur += step_n; r_cur += step_r;
            if (r_cur >= k4) { r_cur -= k4; ++n_cur; }
          }
#pragma unroll
          for (int i = 0; i < BATCH; ++i) {
            if (nn[i] < 0) continue;
            const int n = nn[i];
            const int jc = kk[i] >> 5, w32 = kk[i] & 31;
            unsigned char* dst = wd + size_t(jc) * wd_chunk_bytes + (n >> 3) * 1024 + (n & 7) * 128 +
                                 ((((w32 >> 2) ^ (n & 7))) << 4);
            *reinterpret_cast<float4*>(dst) = make_float4(round_tf32(fmaf(s, ev[i].x, wv[i].x)), round_tf32(fmaf(s, ev[i].y, wv[i].y)),
                                                          round_tf32(fmaf(s, ev[i].z, wv[i].z)), round_tf32(fmaf(s, ev[i].w, wv[i].w)));
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(wd_ready);

      if (drains) {
        for (long long r = r0; r < r1 && ok; ++r) {
          const long long b = r * p.D + d;
          for (int ti = 0; ti < p.tiles_img && ok; ++ti, ++t) {
              const uint32_t buf = t & 1;
              if (!mbar_wait_relaxed(&acc_full[buf], (t >> 1) & 1, 3)) { ok = false; break; }
              tc_fence_after();
              const int qpos = ti * 128 + pix;
              const int oy = qpos / p.Wp, ox = qpos - oy * p.Wp;
              const bool valid = (oy < p.Ho) && (ox < p.Wo) && (timeouts_so_far() == timeouts_at_start);
              float* yb = p.y + size_t(b) * p.Cout * HoWo + size_t(oy) * p.Wo + ox;
              for (int c0 = 0; c0 < p.Cout; c0 += 32) {
                uint32_t acc[32];
                tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + buf * uint32_t(p.Cout) + uint32_t(c0), acc);
                if (valid) {
#pragma unroll
                  for (int j = 0; j < 32; ++j) yb[size_t(c0 + j) * HoWo] = __uint_as_float(acc[j]) + add_s[c0 + j];
                }
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
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// x (B,C,H,W) -> the staged layout the kernel above copies from: for every image and 32-channel chunk a
// run of img_rows pixel rows (zero-padded image, pitch Wp, 128 bytes = 32 channels per row), values rounded
// to TF32, 16-byte groups of each row permuted by (row mod 8) exactly as the 128-byte shared-memory swizzle
// does.
constexpr int STAGE_WARPS = 8;

// One warp per (image, chunk, padded image row, run of 32 pixels), no block-wide synchronisation: a lane reads its pixel
// from the 32 channel planes (32 coalesced 128-byte loads per warp in flight together), rounds to TF32 and writes its
// 128-byte row into the warp's shared-memory tile; the warp reads the tile back so that eight consecutive lanes hold
// one row and stores four whole rows (512 contiguous bytes) per instruction.
__global__ void __launch_bounds__(STAGE_WARPS * 32) stage_rows_tf32_kernel(const float* __restrict__ x, uint4* __restrict__ out,
                                                                         int C, int H, int W, int Hp, int Wp, int ph, int pw,
                                                                         int cchunks, int img_rows, int runs, long long jobs) {
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
        for (int i = lane; i < Wp * 8; i += 32) drow[i] = zero;
      continue;
    }
    if (xr == 0)
      for (int i = lane; i < pw * 8; i += 32) {            // the padding pixels left and right of the row
        drow[i] = zero;
        drow[size_t(pw + W) * 8 + i] = zero;
      }
    const int x0 = xr * 32;
    const int xx = x0 + lane;
    const bool valid = xx < W;
    const float* src = x + ((size_t(b) * C + size_t(cc) * 32) * H + yy) * W + xx;
    float v[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) v[c] = valid ? __ldcs(src + size_t(c) * plane) : 0.f;
    const int row0 = yp * Wp + pw + x0;                // staged row of the run's first pixel (img_rows is a multiple of 8)
    uint4* d0 = drow + size_t(pw + x0) * 8;
#pragma unroll
    for (int g = 0; g < 8; ++g)
      tile[lane * 8 + (g ^ (lane & 7))] = make_uint4(__float_as_uint(round_tf32(v[4 * g])), __float_as_uint(round_tf32(v[4 * g + 1])),
                                                      __float_as_uint(round_tf32(v[4 * g + 2])), __float_as_uint(round_tf32(v[4 * g + 3])));
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = (lane >> 3) + 4 * it;              // pixel of the run; eight lanes per row
      const int pos = lane & 7;                        // 16-byte position in the staged row
      const int chunk = pos ^ ((row0 + r) & 7);        // the channel group that belongs there
      const uint4 val = tile[r * 8 + (chunk ^ (r & 7))];
      if (x0 + r < W) d0[size_t(r) * 8 + pos] = val;
    }
    __syncwarp();
  }
}

// (N, C, ksz) -> (N, ksz, C): the K order the tensor-core kernel uses (k = tap * C + c)
__global__ void reorder_filter_kernel(const float* __restrict__ src, float* __restrict__ dst, int N, int C, int ksz) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= N * C * ksz) return;
  const int n = idx / (C * ksz);
  const int rem = idx - n * C * ksz;
  const int tap = rem / C, c = rem - tap * C;
  dst[idx] = src[(size_t(n) * C + c) * ksz + tap];
}

int conv_tc_error_word(int* v, bool clear) { return read_error_word(v, clear, "tc_error_flag"); }

static int64_t align256(int64_t v) { return (v + 255) & ~int64_t(255); }

struct ConvTcPlan { ConvTcParams p; size_t smem; int64_t x_bytes, map_bytes, filt_bytes; };

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
  p.Hp = H + 2 * ph; p.Wp = W + 2 * pw;
  p.tiles_img = ceil_div(p.Ho * p.Wp, 128);
  const int max_shift = (kh - 1) * dh * p.Wp + (kw - 1) * dw;
  const int rows_needed = 128 + max_shift;
  p.img_rows = (p.Hp * p.Wp + 7) & ~7;            // image stride in rows: keeps (row mod 8) aligned with the tiles
  p.load_bytes = rows_needed * 128;
  p.stage_bytes = (p.load_bytes + 1023) & ~1023;
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
  const size_t table_bytes = (((2 * (size_t(Cout) + Cin)) + 15) & ~size_t(15)) + 4 * size_t(Cout);
  const size_t fixed = 1024 + wd_bytes + 64 /* barriers */ + 16 + 16 + 2 * table_bytes + 8 * size_t(kh) * kw;
  const size_t limit = 227 * 1024;
  NES_REQUIRE(fixed + 2 * (size_t(p.stage_bytes) + 16) <= limit, NES_ERR_UNSUPPORTED,
              "%s: the member filter (%zu bytes) plus two input stages (%d bytes each) do not fit in shared memory on the "
              "tensor-core path", what, wd_bytes, p.stage_bytes);
  int stages = int((limit - fixed) / (size_t(p.stage_bytes) + 16));
  if (stages > 8) stages = 8;
  p.stages = stages;
  pl.smem = 1024 + wd_bytes + size_t(stages) * p.stage_bytes + (2 * stages + 7) * sizeof(uint64_t) + 16 + 16 + 2 * table_bytes + 8 * size_t(kh) * kw;
  pl.x_bytes = align256(D * R * int64_t(p.cchunks) * p.img_rows * 128 + int64_t(p.stage_bytes));
  pl.map_bytes = align256(D * (int64_t(Cin) + Cout) * 2);
  pl.filt_bytes = align256(int64_t(Cout) * Cin * kh * kw * 4);
  return NES_OK;
}

static int run_conv_tc(ConvTcPlan& pl, const float* x, float* x_nhwc, cudaStream_t st, const char* what) {
  ConvTcParams& p = pl.p;
  const int64_t B = p.D * p.R;
  const int runs = ceil_div(p.W, 32);
  const long long jobs = B * int64_t(p.cchunks) * p.Hp * runs;          // one warp per (image, chunk, padded row, 32 pixels)
  long long sblocks = (jobs + STAGE_WARPS - 1) / STAGE_WARPS;
  if (sblocks > 16LL * sm_count()) sblocks = 16LL * sm_count();
  if (sblocks < 1) sblocks = 1;
  stage_rows_tf32_kernel<<<(unsigned)sblocks, STAGE_WARPS * 32, 0, st>>>(x, reinterpret_cast<uint4*>(x_nhwc), p.Cin, p.H, p.W, p.Hp, p.Wp,
                                                                        p.ph, p.pw, p.cchunks, p.img_rows, runs, jobs);
  int rc = check_launch(what);
  if (rc != NES_OK) return rc;

  cudaError_t e = cudaFuncSetAttribute(conv_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "%s: shared memory opt-in failed: %s", what, cudaGetErrorString(e));
  int grid = p.units < sm_count() ? p.units : sm_count();
  if (grid < 1) grid = 1;
  conv_tf32_kernel<<<grid, CONV_THREADS, pl.smem, st>>>(x_nhwc, p);
  return check_launch(what);
}

}  // namespace tc
}  // namespace nes

using namespace nes;
using namespace nes::tc;

extern "C" int64_t nes_conv2d_fwd_tc_scratch_bytes(int64_t D, int64_t R, int Cin, int H, int W, int Cout, int kh, int kw,
                                                   int ph, int pw) {
  if (D <= 0 || R <= 0) return 0;
  const int64_t hp = H + 2 * ph, wp = W + 2 * pw;
  const int64_t img_rows = (hp * wp + 7) & ~int64_t(7);
  const int64_t tail = ((128 + (kh - 1) * wp * 8 + (kw - 1) * 8) * 128 + 1023) & ~int64_t(1023);   // covers any dilation <= 8
  return align256(D * R * int64_t(Cin / 32) * img_rows * 128 + tail) + align256(D * (int64_t(Cin) + Cout) * 2) +
         2 * align256(int64_t(Cout) * Cin * kh * kw * 4);
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
  pl.p.weight_t = nullptr; pl.p.noise_t = nullptr; pl.p.identity_in = 1;
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
  const int64_t need = pl.x_bytes + pl.map_bytes + 2 * pl.filt_bytes;
  NES_REQUIRE(scratch && scratch_bytes >= need && (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0,
              NES_ERR_SCRATCH, "permuted_conv2d_fwd_tc: scratch needs %lld bytes, 256-byte aligned", (long long)need);
  cudaStream_t st = as_stream(stream);
  unsigned char* sp = static_cast<unsigned char*>(scratch);
  int16_t* omap = reinterpret_cast<int16_t*>(sp + pl.x_bytes);
  int16_t* imap = omap + D * Cout;
  float* weight_t = reinterpret_cast<float*>(sp + pl.x_bytes + pl.map_bytes);
  float* eps_t = reinterpret_cast<float*>(sp + pl.x_bytes + pl.map_bytes + pl.filt_bytes);
  rc = launch_permuted_maps(pin, pout, omap, imap, D, Cin, Cout, in_sp, out_sp, st);
  if (rc != NES_OK) return rc;
  const int ksz = kh * kw;
  reorder_filter_kernel<<<ceil_div(Cout * Cin * ksz, 256), 256, 0, st>>>(weight, weight_t, Cout, Cin, ksz);
  if ((rc = check_launch("permuted_conv2d_fwd_tc(reorder W)")) != NES_OK) return rc;
  if (out_sp * in_sp > 0) {
    reorder_filter_kernel<<<ceil_div(out_sp * in_sp * ksz, 256), 256, 0, st>>>(eps, eps_t, out_sp, in_sp, ksz);
    if ((rc = check_launch("permuted_conv2d_fwd_tc(reorder eps)")) != NES_OK) return rc;
  }
  pl.p.weight = weight; pl.p.bias = bias; pl.p.bias_noise = bias_noise; pl.p.y = y;
  pl.p.noise_kind = 2; pl.p.noise = eps; pl.p.omap = omap; pl.p.imap = imap; pl.p.in_sp = in_sp;
  pl.p.weight_t = weight_t; pl.p.noise_t = eps_t; pl.p.identity_in = (pin == nullptr) ? 1 : 0;
  return run_conv_tc(pl, x, static_cast<float*>(scratch), st, "permuted_conv2d_fwd_tc");
}

