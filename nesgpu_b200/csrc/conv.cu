// fp32 NCHW convolutions as implicit GEMMs: plain, dense per-member noise, shared noise with
// member permutations.  One thread block owns 128 output pixels of ONE image, so the whole
// tile belongs to one member and one antithetic sign; the member's effective filter
// W + s*E_d is formed while the B tile is loaded (never materialised in HBM), and the
// GEMM has the unperturbed layer's N = Cout.
#include "gemm_simt.cuh"

namespace nes {
using namespace simt;

struct ConvGeom {
  int Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, Ho, Wo, K, ksz;
};

// per-k decode table kept in shared memory: offset of tap (c,i,j) inside an image and its
// row / column displacement
struct KEntry { int xoff; int dy; int dx; int c_tap; };  // c_tap = c << 12 | tap

// ---- noise policies for the B (filter) tile ---------------------------------------------
struct NoNoise {
  __device__ inline float operator()(int64_t, int, int, const KEntry&) const { return 0.f; }
};
struct DenseNoise {   // noise (D, Cout, K)
  const float* E; int Cout; int K;
  __device__ inline float operator()(int64_t d, int n, int k, const KEntry&) const {
    return __ldg(E + (size_t(d) * Cout + n) * K + k);
  }
};
struct PermutedNoise {  // eps (out_sp, in_sp, ksz); omap (D,Cout), imap (D,Cin): -1 = no noise
  const float* eps; const int16_t* omap; const int16_t* imap; int Cout, Cin, in_sp, ksz;
  __device__ inline float operator()(int64_t d, int n, int, const KEntry& e) const {
    const int so = omap[d * Cout + n];
    const int ci = imap[d * Cin + (e.c_tap >> 12)];
    if (so < 0 || ci < 0) return 0.f;
    return __ldg(eps + (size_t(so) * in_sp + ci) * ksz + (e.c_tap & 4095));
  }
};

struct SyntheticNoise {  // eps (Cout, Cin, ksz) times the member's output / input channel signs (+-1 int8, NULL = +1)
  const float* eps; const int8_t* fout; const int8_t* fin; int Cout, Cin, K;
  __device__ inline float operator()(int64_t d, int n, int k, const KEntry& e) const {
    float v = __ldg(eps + size_t(n) * K + k);
    if (fout) v *= float(fout[d * Cout + n]);
    if (fin) v *= float(fin[d * Cin + (e.c_tap >> 12)]);
    return v;
  }
};

template <class Noise, int NJ_>
struct ConvProb {
  static constexpr bool MFAST = true;
  static constexpr int NJ = NJ_;
  static constexpr int TN = 64 * NJ_;
  ConvGeom g; Noise noise;
  const float* x; const float* weight; const float* bias; const float* bias_noise; float* y;
  int64_t D, R; int antithetic; int tiles_per_img; int vec_store;

  struct Ctx {
    const KEntry* ktab; const float* ximg; int64_t b, d; float s;
    int m0, n0; int iy0, ix0; bool pix_ok;
  };
  __device__ inline int k_extent() const { return g.K; }

  __device__ inline void init(Ctx& c) const {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    KEntry* tab = reinterpret_cast<KEntry*>(dyn_smem);
    for (int k = threadIdx.x; k < g.K; k += NT) {
      const int ch = k / g.ksz, tap = k - ch * g.ksz;
      const int i = tap / g.kw, j = tap - i * g.kw;
      KEntry e; e.dy = i * g.dh; e.dx = j * g.dw;
      e.xoff = (ch * g.H + e.dy) * g.W + e.dx; e.c_tap = (ch << 12) | tap;
      tab[k] = e;
    }
    __syncthreads();
    c.ktab = tab;
    c.b = blockIdx.x / tiles_per_img;
    c.m0 = (blockIdx.x - c.b * tiles_per_img) * BM;
    c.n0 = blockIdx.y * TN;
    c.d = c.b % D;
    c.s = anti_sign(c.b / D, R, antithetic);
    c.ximg = x + size_t(c.b) * g.Cin * g.H * g.W;
    const int pm = c.m0 + (threadIdx.x & 127);
    c.pix_ok = pm < g.Ho * g.Wo;
    const int oy = pm / g.Wo, ox = pm - oy * g.Wo;
    c.iy0 = oy * g.sh - g.ph;
    c.ix0 = ox * g.sw - g.pw;
  }

  // A: im2col patches.  Thread t owns pixel t%128 and k = k0 + t/128 + 2*i.
  __device__ inline void fetchA(const Ctx& c, int k0, Frag& f) const {
    const int kb = k0 + (threadIdx.x >> 7);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = kb + 2 * i;
      float v = 0.f;
      if (c.pix_ok && k < g.K) {
        const KEntry e = c.ktab[k];
        const int iy = c.iy0 + e.dy, ix = c.ix0 + e.dx;
        if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) v = __ldg(c.ximg + e.xoff + c.iy0 * g.W + c.ix0);
      }
      f.v[i] = v;
    }
  }
  __device__ inline void storeA(TilePtr T, const Frag& f) const {
    const int m = threadIdx.x & 127, kb = threadIdx.x >> 7;
#pragma unroll
    for (int i = 0; i < 8; ++i) T[kb + 2 * i][m] = f.v[i];
  }
  // B: effective filter rows.  Thread t owns k = k0 + t%16 and filters n0 + t/16 + 16*i.
  __device__ inline void fetchB(const Ctx& c, int k0, Frag& f) const {
    const int k = k0 + (threadIdx.x & 15);
    KEntry e; e.xoff = e.dy = e.dx = e.c_tap = 0;
    if (k < g.K) e = c.ktab[k];
#pragma unroll
    for (int i = 0; i < TN / 16; ++i) {
      const int n = c.n0 + (threadIdx.x >> 4) + 16 * i;
      float v = 0.f;
      if (n < g.Cout && k < g.K) v = __ldg(weight + size_t(n) * g.K + k) + c.s * noise(c.d, n, k, e);
      f.v[i] = v;
    }
  }
  __device__ inline void storeB(TilePtr T, const Frag& f) const { store_elementwise<TN>(T, f); }

  __device__ inline void epilogue(const Ctx& c, float (&acc)[8][4 * NJ_], int tm, int tn) const {
    const int HoWo = g.Ho * g.Wo;
#pragma unroll
    for (int jg = 0; jg < NJ_; ++jg) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = c.n0 + jg * 64 + tn * 4 + j;
        if (n >= g.Cout) continue;
        float add = bias ? __ldg(bias + n) : 0.f;
        if (bias_noise) add += c.s * __ldg(bias_noise + c.d * g.Cout + n);
        float* plane = y + (size_t(c.b) * g.Cout + n) * HoWo;
#pragma unroll
        for (int ig = 0; ig < 2; ++ig) {
          const int pm = c.m0 + ig * 64 + tm * 4;
          const int a = ig * 4;
          if (vec_store && pm + 3 < HoWo) {
            *reinterpret_cast<float4*>(plane + pm) = make_float4(
                acc[a][jg * 4 + j] + add, acc[a + 1][jg * 4 + j] + add,
                acc[a + 2][jg * 4 + j] + add, acc[a + 3][jg * 4 + j] + add);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) if (pm + i < HoWo) plane[pm + i] = acc[a + i][jg * 4 + j] + add;
          }
        }
      }
    }
  }
};

static int make_geom(ConvGeom& g, int Cin, int H, int W, int Cout, int kh, int kw, int sh, int sw,
                     int ph, int pw, int dh, int dw, const char* what) {
  NES_REQUIRE(Cin > 0 && H > 0 && W > 0 && Cout > 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0 &&
              ph >= 0 && pw >= 0 && dh > 0 && dw > 0, NES_ERR_BAD_ARG, "%s: bad geometry", what);
  g.Cin = Cin; g.H = H; g.W = W; g.Cout = Cout; g.kh = kh; g.kw = kw; g.sh = sh; g.sw = sw;
  g.ph = ph; g.pw = pw; g.dh = dh; g.dw = dw;
  g.Ho = (H + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
  g.Wo = (W + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
  g.ksz = kh * kw; g.K = Cin * g.ksz;
  NES_REQUIRE(g.Ho > 0 && g.Wo > 0, NES_ERR_BAD_ARG, "%s: empty output", what);
  NES_REQUIRE(g.ksz < 4096 && Cin < (1 << 19), NES_ERR_UNSUPPORTED, "%s: kernel window or channel count too large", what);
  NES_REQUIRE(size_t(g.K) * sizeof(KEntry) <= 160 * 1024, NES_ERR_UNSUPPORTED,
              "%s: Cin*kh*kw = %d exceeds the shared-memory decode table (10240)", what, g.K);
  NES_REQUIRE(int64_t(Cin) * H * W < INT32_MAX, NES_ERR_UNSUPPORTED, "%s: image too large", what);
  return NES_OK;
}

template <class Noise, int NJ_>
static int launch_conv_nj(const ConvGeom& g, const Noise& noise, const float* x, const float* weight,
                          const float* bias, const float* bias_noise, float* y, int64_t D, int64_t R,
                          int antithetic, cudaStream_t st, const char* what) {
  ConvProb<Noise, NJ_> p;
  p.g = g; p.noise = noise; p.x = x; p.weight = weight; p.bias = bias; p.bias_noise = bias_noise; p.y = y;
  p.D = D; p.R = R; p.antithetic = antithetic;
  const int HoWo = g.Ho * g.Wo;
  p.tiles_per_img = ceil_div(HoWo, BM);
  p.vec_store = (HoWo % 4 == 0) && aligned16(y);
  const int64_t B = D * R;
  const int64_t gx = B * p.tiles_per_img;
  NES_REQUIRE(gx <= INT32_MAX, NES_ERR_UNSUPPORTED, "%s: too many tiles", what);
  const size_t smem = size_t(g.K) * sizeof(KEntry);
  auto kern = gemm_kernel<ConvProb<Noise, NJ_>>;
  if (smem + 2 * 2 * BK * LDS * sizeof(float) > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(NES_ERR_UNSUPPORTED, "%s: %zu B of dynamic shared memory refused", what, smem);
  }
  dim3 grid((unsigned)gx, (unsigned)ceil_div(g.Cout, 64 * NJ_));
  kern<<<grid, NT, smem, st>>>(p);
  return check_launch(what);
}

template <class Noise>
static int launch_conv(const ConvGeom& g, const Noise& noise, const float* x, const float* weight,
                       const float* bias, const float* bias_noise, float* y, int64_t D, int64_t R,
                       int antithetic, cudaStream_t st, const char* what) {
  if (g.Cout <= 64) return launch_conv_nj<Noise, 1>(g, noise, x, weight, bias, bias_noise, y, D, R, antithetic, st, what);
  return launch_conv_nj<Noise, 2>(g, noise, x, weight, bias, bias_noise, y, D, R, antithetic, st, what);
}

// omap[d,k] = pout[d,k] if < out_sp else -1 (identity without output permutation);
// imap[d,c] = j with pin[d,j] == c, else -1 (identity without input permutation).
__global__ void permuted_maps_kernel(const int16_t* pin, const int16_t* pout, int16_t* omap, int16_t* imap,
                                     int64_t D, int Cin, int Cout, int in_sp, int out_sp) {
  const int64_t d = blockIdx.x;
  for (int k = threadIdx.x; k < Cout; k += blockDim.x) {
    const int so = pout ? int(pout[d * Cout + k]) : k;
    omap[d * Cout + k] = (so < out_sp) ? int16_t(so) : int16_t(-1);
  }
  for (int c = threadIdx.x; c < Cin; c += blockDim.x) imap[d * Cin + c] = pin ? int16_t(-1) : int16_t(c);
  __syncthreads();
  if (pin)
    for (int j = threadIdx.x; j < in_sp; j += blockDim.x) imap[d * Cin + pin[d * in_sp + j]] = int16_t(j);
}

// E[d,k,m,t] = sum_j [pin[d,j]==m] eps[pout[d,k], j, t]
__global__ void permuted_dense_noise_kernel(const float* __restrict__ eps, const int16_t* __restrict__ pin,
                                            const int16_t* __restrict__ pout, float* __restrict__ E,
                                            int in, int out, int in_sp, int out_sp, int ksz) {
  const int64_t d = blockIdx.y;
  const int k = blockIdx.x;
  float* row = E + (size_t(d) * out + k) * in * ksz;
  for (int e = threadIdx.x; e < in * ksz; e += blockDim.x) row[e] = 0.f;
  __syncthreads();
  const int so = pout ? int(pout[d * out + k]) : k;
  if (so >= out_sp) return;
  const float* src = eps + size_t(so) * in_sp * ksz;
  if (!pin) {
    for (int e = threadIdx.x; e < in_sp * ksz; e += blockDim.x) row[e] = src[e];
  } else {
    for (int e = threadIdx.x; e < in_sp * ksz; e += blockDim.x) {
      const int j = e / ksz, t = e - j * ksz;
      atomicAdd(row + int(pin[d * in_sp + j]) * ksz + t, src[e]);   // repeated inputs add
    }
  }
}

// host-side launcher shared with the tensor-core path (conv_tc.cu)
int launch_permuted_maps(const int16_t* pin, const int16_t* pout, int16_t* omap, int16_t* imap, int64_t D,
                         int Cin, int Cout, int in_sp, int out_sp, cudaStream_t st) {
  NES_REQUIRE(Cin <= 32767 && Cout <= 32767 && D <= INT32_MAX, NES_ERR_UNSUPPORTED, "permuted maps: degree > 32767");
  permuted_maps_kernel<<<(unsigned)D, 128, 0, st>>>(pin, pout, omap, imap, D, Cin, Cout, in_sp, out_sp);
  return check_launch("permuted_conv2d_fwd(maps)");
}

}  // namespace nes

using namespace nes;

extern "C" int nes_conv2d_fwd(const float* x, const float* weight, const float* bias, float* y,
                              int64_t B, int Cin, int H, int W, int Cout, int kh, int kw,
                              int sh, int sw, int ph, int pw, int dh, int dw, nes_stream_t stream) {
  NES_REQUIRE(B >= 0, NES_ERR_BAD_ARG, "conv2d_fwd: negative batch");
  if (B == 0) return NES_OK;
  NES_REQUIRE(x && weight && y, NES_ERR_BAD_ARG, "conv2d_fwd: null pointer");
  ConvGeom g;
  int rc = make_geom(g, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, "conv2d_fwd");
  if (rc != NES_OK) return rc;
  return launch_conv(g, NoNoise(), x, weight, bias, nullptr, y, B, 1, 0, as_stream(stream), "conv2d_fwd");
}

extern "C" int nes_perturbed_conv2d_fwd(const float* x, const float* weight, const float* bias,
                                        const float* noise, const float* bias_noise, float* y,
                                        int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                        int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                        int antithetic, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0, NES_ERR_BAD_ARG, "perturbed_conv2d_fwd: negative extent");
  if (D == 0 || R == 0) return NES_OK;
  NES_REQUIRE(x && weight && noise && y, NES_ERR_BAD_ARG, "perturbed_conv2d_fwd: null pointer");
  ConvGeom g;
  int rc = make_geom(g, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, "perturbed_conv2d_fwd");
  if (rc != NES_OK) return rc;
  DenseNoise n; n.E = noise; n.Cout = Cout; n.K = g.K;
  return launch_conv(g, n, x, weight, bias, bias_noise, y, D, R, antithetic, as_stream(stream), "perturbed_conv2d_fwd");
}

extern "C" int64_t nes_permuted_conv2d_fwd_scratch_bytes(int64_t D, int Cin, int Cout) {
  return D * (int64_t(Cin) + Cout) * (int64_t)sizeof(int16_t);
}

extern "C" int nes_permuted_conv2d_fwd(const float* x, const float* weight, const float* bias,
                                       const float* eps, const float* bias_noise,
                                       const int16_t* pin, const int16_t* pout, float* y,
                                       int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                       int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                       int in_sp, int out_sp, int antithetic,
                                       void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0, NES_ERR_BAD_ARG, "permuted_conv2d_fwd: negative extent");
  if (D == 0 || R == 0) return NES_OK;
  NES_REQUIRE(x && weight && eps && y, NES_ERR_BAD_ARG, "permuted_conv2d_fwd: null pointer");
  NES_REQUIRE(out_sp >= 0 && out_sp <= Cout && in_sp >= 0 && in_sp <= Cin, NES_ERR_BAD_ARG,
              "permuted_conv2d_fwd: sparsity exceeds degree");
  NES_REQUIRE(pin || in_sp == Cin, NES_ERR_BAD_ARG, "permuted_conv2d_fwd: in_sp != Cin without input permutations");
  NES_REQUIRE(Cin <= 32767 && Cout <= 32767 && D <= INT32_MAX, NES_ERR_UNSUPPORTED, "permuted_conv2d_fwd: degree > 32767");
  NES_REQUIRE(scratch && scratch_bytes >= nes_permuted_conv2d_fwd_scratch_bytes(D, Cin, Cout), NES_ERR_SCRATCH,
              "permuted_conv2d_fwd: scratch needs %lld bytes", (long long)nes_permuted_conv2d_fwd_scratch_bytes(D, Cin, Cout));
  ConvGeom g;
  int rc = make_geom(g, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, "permuted_conv2d_fwd");
  if (rc != NES_OK) return rc;
  cudaStream_t st = as_stream(stream);
  int16_t* omap = static_cast<int16_t*>(scratch);
  int16_t* imap = omap + D * Cout;
  rc = launch_permuted_maps(pin, pout, omap, imap, D, Cin, Cout, in_sp, out_sp, st);
  if (rc != NES_OK) return rc;
  PermutedNoise n; n.eps = eps; n.omap = omap; n.imap = imap; n.Cout = Cout; n.Cin = Cin; n.in_sp = in_sp; n.ksz = g.ksz;
  return launch_conv(g, n, x, weight, bias, bias_noise, y, D, R, antithetic, st, "permuted_conv2d_fwd");
}

extern "C" int nes_permuted_dense_noise(const float* eps, const int16_t* pin, const int16_t* pout, float* E,
                                        int64_t D, int in, int out, int in_sp, int out_sp, int ksize,
                                        nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && in > 0 && out > 0 && in_sp >= 0 && out_sp >= 0 && ksize > 0, NES_ERR_BAD_ARG,
              "permuted_dense_noise: bad extent");
  if (D == 0) return NES_OK;
  NES_REQUIRE(eps && E, NES_ERR_BAD_ARG, "permuted_dense_noise: null pointer");
  NES_REQUIRE(out_sp <= out && (pin || in_sp == in), NES_ERR_BAD_ARG, "permuted_dense_noise: sparsity exceeds degree");
  NES_REQUIRE(D <= 65535, NES_ERR_UNSUPPORTED, "permuted_dense_noise: D > 65535");
  dim3 grid((unsigned)out, (unsigned)D);
  permuted_dense_noise_kernel<<<grid, 128, 0, as_stream(stream)>>>(eps, pin, pout, E, in, out, in_sp, out_sp, ksize);
  return check_launch("permuted_dense_noise");
}

extern "C" int nes_synthetic_conv2d_fwd(const float* x, const float* weight, const float* bias,
                                        const float* eps, const float* bias_noise,
                                        const int8_t* fin, const int8_t* fout, float* y,
                                        int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                        int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                        int antithetic, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0, NES_ERR_BAD_ARG, "synthetic_conv2d_fwd: negative extent");
  if (D == 0 || R == 0) return NES_OK;
  NES_REQUIRE(x && weight && eps && y, NES_ERR_BAD_ARG, "synthetic_conv2d_fwd: null pointer");
  ConvGeom g;
  int rc = make_geom(g, Cin, H, W, Cout, kh, kw, sh, sw, ph, pw, dh, dw, "synthetic_conv2d_fwd");
  if (rc != NES_OK) return rc;
  SyntheticNoise n; n.eps = eps; n.fout = fout; n.fin = fin; n.Cout = Cout; n.Cin = Cin; n.K = g.K;
  return launch_conv(g, n, x, weight, bias, bias_noise, y, D, R, antithetic, as_stream(stream), "synthetic_conv2d_fwd");
}
