// fp32 linear layers: plain, dense per-member noise (streaming), shared noise with member
// permutations, sparse per-member noise.
#include "gemm_simt.cuh"

namespace nes {
using namespace simt;

// ---- epilogues ------------------------------------------------------------------------

struct BiasEpi {
  const float* bias;
  struct Row {};
  __device__ inline Row row(int64_t) const { return Row(); }
  __device__ inline float operator()(const Row&, int64_t, int gn, float acc) const {
    return bias ? acc + __ldg(bias + gn) : acc;
  }
};

// y = acc + bias + s(r) * (p[b, pout[d,k]] + bias_noise[d,k])      (modules/base.py:501-506)
struct PermutedEpi {
  const float* bias; const float* p; const int16_t* pout; const float* bias_noise;
  int64_t D, R; int N; int out_sp; int antithetic;
  struct Row { int64_t d; float s; };
  __device__ inline Row row(int64_t gm) const {
    Row r; r.d = gm % D; r.s = anti_sign(gm / D, R, antithetic); return r;
  }
  __device__ inline float operator()(const Row& r, int64_t gm, int gn, float acc) const {
    const int so = pout ? int(pout[r.d * N + gn]) : gn;
    float q = (so < out_sp) ? __ldg(p + gm * out_sp + so) : 0.f;
    if (bias_noise) q += __ldg(bias_noise + r.d * N + gn);
    float v = acc + r.s * q;
    return bias ? v + __ldg(bias + gn) : v;
  }
};

// y = acc + bias + s(r) * (p[b,k] * fout[d,k] + bias_noise[d,k])      (modules/base.py:620-626)
struct FlipEpi {
  const float* bias; const float* p; const int8_t* fout; const float* bias_noise;
  int64_t D, R; int N; int antithetic;
  struct Row { int64_t d; float s; };
  __device__ inline Row row(int64_t gm) const {
    Row r; r.d = gm % D; r.s = anti_sign(gm / D, R, antithetic); return r;
  }
  __device__ inline float operator()(const Row& r, int64_t gm, int gn, float acc) const {
    float q = __ldg(p + gm * N + gn);
    if (fout) q *= float(fout[r.d * N + gn]);
    if (bias_noise) q += __ldg(bias_noise + r.d * N + gn);
    float v = acc + r.s * q;
    return bias ? v + __ldg(bias + gn) : v;
  }
};

// y = acc + bias + s(r) * (sum_t x[b, idx[d,o,t]] * val[d,o,t] + bias_noise[d,o])
struct SparseEpi {
  const float* bias; const float* x; const int32_t* idx; const float* val; const float* bias_noise;
  int64_t D, R; int N; int in; int k; int antithetic;
  struct Row { int64_t d; float s; };
  __device__ inline Row row(int64_t gm) const {
    Row r; r.d = gm % D; r.s = anti_sign(gm / D, R, antithetic); return r;
  }
  __device__ inline float operator()(const Row& r, int64_t gm, int gn, float acc) const {
    const int64_t e = (r.d * N + gn) * k;
    float q = 0.f;
    for (int t = 0; t < k; ++t) q = fmaf(__ldg(x + gm * in + idx[e + t]), __ldg(val + e + t), q);
    if (bias_noise) q += __ldg(bias_noise + r.d * N + gn);
    float v = acc + r.s * q;
    return bias ? v + __ldg(bias + gn) : v;
  }
};

// ---- problem: C[M,N] = A[M,K] . W[N,K]^T with a row-major store ------------------------

template <class ALoader, class Epi, int NJ_>
struct LinearProb {
  static constexpr bool MFAST = false;
  static constexpr int NJ = NJ_;
  static constexpr int TN = 64 * NJ_;
  ALoader A; RowsLoader B; Epi epi; float* y; int64_t M; int N; int K; int vec_store;
  struct Ctx { int64_t m0; int n0; };
  __device__ inline void init(Ctx& c) const { c.m0 = int64_t(blockIdx.x) * BM; c.n0 = blockIdx.y * TN; }
  __device__ inline int k_extent() const { return K; }
  __device__ inline void fetchA(const Ctx& c, int k0, Frag& f) const { A.template fetch<BM>(c.m0, k0, f); }
  __device__ inline void fetchB(const Ctx& c, int k0, Frag& f) const { B.template fetch<TN>(c.n0, k0, f); }
  __device__ inline void storeA(TilePtr T, const Frag& f) const { ALoader::template store<BM>(T, f); }
  __device__ inline void storeB(TilePtr T, const Frag& f) const { RowsLoader::template store<TN>(T, f); }
  __device__ inline void epilogue(const Ctx& c, float (&acc)[8][4 * NJ_], int tm, int tn) const {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int64_t gm = c.m0 + micro_index(tm, i);
      if (gm >= M) continue;
      const typename Epi::Row ri = epi.row(gm);
#pragma unroll
      for (int jg = 0; jg < NJ_; ++jg) {
        const int gn0 = c.n0 + jg * 64 + tn * 4;
        float o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = (gn0 + j < N) ? epi(ri, gm, gn0 + j, acc[i][jg * 4 + j]) : 0.f;
        float* dst = y + gm * N + gn0;
        if (vec_store && gn0 + 3 < N) {
          *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) if (gn0 + j < N) dst[j] = o[j];
        }
      }
    }
  }
};

static inline RowsLoader rows_loader(const float* src, int64_t ld, int64_t rows, int K) {
  RowsLoader L; L.src = src; L.ld = ld; L.rows = rows; L.K = K;
  L.vec = (ld % 4 == 0) && aligned16(src);
  return L;
}

template <class ALoader, class Epi>
static int launch_linear(const ALoader& A, const float* weight, const Epi& epi, float* y,
                         int64_t M, int64_t N, int64_t K, cudaStream_t st, const char* what) {
  if (M == 0 || N == 0) return NES_OK;
  NES_REQUIRE(N <= 65535LL * BN && K <= INT32_MAX && M <= int64_t(INT32_MAX) * BM, NES_ERR_UNSUPPORTED,
              "%s: extent too large (M=%lld N=%lld K=%lld)", what, (long long)M, (long long)N, (long long)K);
  if (N <= 64) {
    LinearProb<ALoader, Epi, 1> p;
    p.A = A; p.B = rows_loader(weight, K, N, int(K)); p.epi = epi; p.y = y;
    p.M = M; p.N = int(N); p.K = int(K);
    p.vec_store = (N % 4 == 0) && aligned16(y);
    dim3 grid((unsigned)ceil_div<int64_t>(M, BM), 1);
    gemm_kernel<<<grid, NT, 0, st>>>(p);
  } else {
    LinearProb<ALoader, Epi, 2> p;
    p.A = A; p.B = rows_loader(weight, K, N, int(K)); p.epi = epi; p.y = y;
    p.M = M; p.N = int(N); p.K = int(K);
    p.vec_store = (N % 4 == 0) && aligned16(y);
    dim3 grid((unsigned)ceil_div<int64_t>(M, BM), (unsigned)ceil_div<int64_t>(N, BN));
    gemm_kernel<<<grid, NT, 0, st>>>(p);
  }
  return check_launch(what);
}

// ---- dense per-member noise: streaming kernel -------------------------------------------
//
// The per-member term x[b].E_d^T touches every element of the (D,out,in) noise exactly once
// per pass and does RT multiply-adds per element: HBM-bound.  One block takes 64 output rows
// of one member; each warp streams whole noise rows with 128-bit evict-first loads (eight in
// flight per lane), multiplies them with the member's RT input rows held in shared memory
// and reduces across the warp.  Results are staged in shared memory so that the read of the
// base GEMM result and the write of y are coalesced.
constexpr int STREAM_ROWS = 64;

template <int RT, bool VEC>
__global__ void __launch_bounds__(256) perturbed_linear_stream_kernel(
    const float* __restrict__ x, const float* __restrict__ E, const float* __restrict__ beta,
    float* __restrict__ y, int64_t D, int64_t R, int in, int out, int64_t r0, int antithetic, int direct) {
  extern __shared__ __align__(16) float smem[];
  float* xs = smem;                       // [RT][in]
  float* res = smem + size_t(RT) * in;    // [RT][STREAM_ROWS]
  const int64_t d = blockIdx.y;
  const int o0 = blockIdx.x * STREAM_ROWS;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;

  for (int rr = 0; rr < RT; ++rr) {
    const float* xr = x + ((r0 + rr) * D + d) * in;
    for (int c = t; c < in; c += 256) xs[rr * in + c] = __ldg(xr + c);
  }
  __syncthreads();

  for (int ro = warp; ro < STREAM_ROWS; ro += 8) {
    const int o = o0 + ro;
    if (o >= out) break;
    const float* er = E + (size_t(d) * out + o) * in;
    float acc[RT];
#pragma unroll
    for (int rr = 0; rr < RT; ++rr) acc[rr] = 0.f;
    if (VEC) {
#pragma unroll 8
      for (int c = lane * 4; c < in; c += 128) {
        const float4 e = __ldcs(reinterpret_cast<const float4*>(er + c));
#pragma unroll
        for (int rr = 0; rr < RT; ++rr) {
          const float4 xv = *reinterpret_cast<const float4*>(xs + rr * in + c);
          acc[rr] = fmaf(e.x, xv.x, acc[rr]); acc[rr] = fmaf(e.y, xv.y, acc[rr]);
          acc[rr] = fmaf(e.z, xv.z, acc[rr]); acc[rr] = fmaf(e.w, xv.w, acc[rr]);
        }
      }
    } else {
      for (int c = lane; c < in; c += 32) {
        const float e = __ldcs(er + c);
#pragma unroll
        for (int rr = 0; rr < RT; ++rr) acc[rr] = fmaf(e, xs[rr * in + c], acc[rr]);
      }
    }
#pragma unroll
    for (int rr = 0; rr < RT; ++rr) {
      float v = acc[rr];
#pragma unroll
      for (int sh = 16; sh > 0; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
      if (lane == 0) res[rr * STREAM_ROWS + ro] = v;
    }
  }
  __syncthreads();

  for (int e = t; e < RT * STREAM_ROWS; e += 256) {
    const int rr = e / STREAM_ROWS, ro = e % STREAM_ROWS;
    const int o = o0 + ro;
    if (o >= out) continue;
    float v = res[e];
    if (beta) v += __ldg(beta + d * out + o);
    float* dst = y + ((r0 + rr) * D + d) * out + o;
    if (direct) *dst = v;
    else *dst = *dst + anti_sign(r0 + rr, R, antithetic) * v;
  }
}

template <int RT>
static int launch_stream(const float* x, const float* E, const float* beta, float* y, int64_t D,
                         int64_t R, int64_t in, int64_t out, int64_t r0, int antithetic, int direct,
                         cudaStream_t st) {
  const bool vec = (in % 4 == 0) && aligned16(E) && aligned16(x);
  const size_t smem = (size_t(RT) * in + RT * STREAM_ROWS) * sizeof(float);
  dim3 grid((unsigned)ceil_div<int64_t>(out, STREAM_ROWS), (unsigned)D);
  auto kern = vec ? perturbed_linear_stream_kernel<RT, true> : perturbed_linear_stream_kernel<RT, false>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(NES_ERR_UNSUPPORTED, "perturbed_linear_fwd: in=%lld needs %zu B of shared memory", (long long)in, smem);
  }
  kern<<<grid, 256, smem, st>>>(x, E, beta, y, D, R, int(in), int(out), r0, antithetic, direct);
  return check_launch("perturbed_linear_fwd(stream)");
}

}  // namespace nes

using namespace nes;

extern "C" int nes_linear_fwd(const float* x, const float* weight, const float* bias, float* y,
                              int64_t M, int64_t N, int64_t K, nes_stream_t stream) {
  NES_REQUIRE(M >= 0 && N >= 0 && K >= 0, NES_ERR_BAD_ARG, "linear_fwd: negative extent");
  if (M == 0 || N == 0) return NES_OK;
  NES_REQUIRE(x && weight && y, NES_ERR_BAD_ARG, "linear_fwd: null pointer");
  BiasEpi epi; epi.bias = bias;
  return launch_linear(rows_loader(x, K, M, int(K)), weight, epi, y, M, N, K, as_stream(stream), "linear_fwd");
}

extern "C" int nes_perturbed_linear_fwd(const float* x, const float* weight, const float* bias,
                                        const float* noise, const float* bias_noise, float* y,
                                        int64_t D, int64_t R, int64_t in, int64_t out,
                                        int antithetic, int direct, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0 && in >= 0 && out >= 0, NES_ERR_BAD_ARG, "perturbed_linear_fwd: negative extent");
  if (D == 0 || R == 0 || out == 0) return NES_OK;
  NES_REQUIRE(x && noise && y && (direct != 0 || weight), NES_ERR_BAD_ARG, "perturbed_linear_fwd: null pointer");
  NES_REQUIRE(D <= 65535, NES_ERR_UNSUPPORTED, "perturbed_linear_fwd: D=%lld > 65535", (long long)D);
  NES_REQUIRE(in <= 48000, NES_ERR_UNSUPPORTED, "perturbed_linear_fwd: in=%lld > 48000", (long long)in);
  cudaStream_t st = as_stream(stream);
  NES_REQUIRE(direct >= 0 && direct <= 2, NES_ERR_BAD_ARG, "perturbed_linear_fwd: direct must be 0, 1 or 2");
  if (direct == 0) {
    int rc = nes_linear_fwd(x, weight, bias, y, D * R, out, in, stream);
    if (rc != NES_OK) return rc;
  }
  if (direct == 2) direct = 0;   // y already holds x.W^T + bias: only the per-member term is added
  int64_t r0 = 0;
  while (r0 < R) {
    const int64_t left = R - r0;
    int rc;
    if (left >= 4 && in <= 12000) { rc = launch_stream<4>(x, noise, bias_noise, y, D, R, in, out, r0, antithetic, direct, st); r0 += 4; }
    else if (left >= 2 && in <= 24000) { rc = launch_stream<2>(x, noise, bias_noise, y, D, R, in, out, r0, antithetic, direct, st); r0 += 2; }
    else { rc = launch_stream<1>(x, noise, bias_noise, y, D, R, in, out, r0, antithetic, direct, st); r0 += 1; }
    if (rc != NES_OK) return rc;
  }
  return NES_OK;
}

extern "C" int64_t nes_permuted_linear_fwd_scratch_bytes(int64_t D, int64_t R, int64_t out_sp) {
  return D * R * out_sp * (int64_t)sizeof(float);
}

extern "C" int nes_permuted_linear_fwd(const float* x, const float* weight, const float* bias,
                                       const float* eps, const float* bias_noise,
                                       const int16_t* pin, const int16_t* pout, float* y,
                                       int64_t D, int64_t R, int64_t in, int64_t out,
                                       int64_t in_sp, int64_t out_sp, int antithetic,
                                       void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0 && in >= 0 && out >= 0 && in_sp >= 0 && out_sp >= 0, NES_ERR_BAD_ARG,
              "permuted_linear_fwd: negative extent");
  if (D == 0 || R == 0 || out == 0) return NES_OK;
  NES_REQUIRE(x && weight && eps && y, NES_ERR_BAD_ARG, "permuted_linear_fwd: null pointer");
  NES_REQUIRE(out_sp <= out && in_sp <= (pin ? INT32_MAX : in), NES_ERR_BAD_ARG, "permuted_linear_fwd: sparsity exceeds degree");
  NES_REQUIRE(pin || in_sp == in, NES_ERR_BAD_ARG, "permuted_linear_fwd: in_sp != in without input permutations");
  NES_REQUIRE(scratch && scratch_bytes >= nes_permuted_linear_fwd_scratch_bytes(D, R, out_sp) && aligned16(scratch),
              NES_ERR_SCRATCH, "permuted_linear_fwd: scratch needs %lld bytes, 16-byte aligned",
              (long long)nes_permuted_linear_fwd_scratch_bytes(D, R, out_sp));
  cudaStream_t st = as_stream(stream);
  const int64_t B = D * R;
  float* p = static_cast<float*>(scratch);
  // 1) p = gather_in(x) . eps^T
  BiasEpi none; none.bias = nullptr;
  int rc;
  if (pin) {
    GatherKLoader g; g.src = x; g.ld = in; g.rows = B; g.K = int(in_sp); g.perm = pin; g.D = D;
    rc = launch_linear(g, eps, none, p, B, out_sp, in_sp, st, "permuted_linear_fwd(noise)");
  } else {
    rc = launch_linear(rows_loader(x, in, B, int(in)), eps, none, p, B, out_sp, in, st, "permuted_linear_fwd(noise)");
  }
  if (rc != NES_OK) return rc;
  // 2) y = x . W^T + bias + s * (gather_out(p) + bias_noise)
  PermutedEpi epi;
  epi.bias = bias; epi.p = p; epi.pout = pout; epi.bias_noise = bias_noise;
  epi.D = D; epi.R = R; epi.N = int(out); epi.out_sp = int(out_sp); epi.antithetic = antithetic;
  return launch_linear(rows_loader(x, in, B, int(in)), weight, epi, y, B, out, in, st, "permuted_linear_fwd(base)");
}

extern "C" int nes_sparse_perturbed_linear_fwd(const float* x, const float* weight, const float* bias,
                                               const int32_t* idx, const float* val, const float* bias_noise,
                                               float* y, int64_t D, int64_t R, int64_t in, int64_t out,
                                               int k, int antithetic, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0 && in >= 0 && out >= 0 && k >= 0, NES_ERR_BAD_ARG, "sparse_perturbed_linear_fwd: negative extent");
  if (D == 0 || R == 0 || out == 0) return NES_OK;
  NES_REQUIRE(x && weight && y && (k == 0 || (idx && val)), NES_ERR_BAD_ARG, "sparse_perturbed_linear_fwd: null pointer");
  SparseEpi epi;
  epi.bias = bias; epi.x = x; epi.idx = idx; epi.val = val; epi.bias_noise = bias_noise;
  epi.D = D; epi.R = R; epi.N = int(out); epi.in = int(in); epi.k = k; epi.antithetic = antithetic;
  return launch_linear(rows_loader(x, in, D * R, int(in)), weight, epi, y, D * R, out, in,
                       as_stream(stream), "sparse_perturbed_linear_fwd");
}

// y[i] = x[i] * scale[i % period] + shift[i % period]: per-member scale and shift broadcast over the leading
// dimensions of x (PerturbedAffine.forward, modules/base.py:437-444)
__global__ void affine_kernel(const float* __restrict__ x, const float* __restrict__ scale, const float* __restrict__ shift,
                              float* __restrict__ y, int64_t n, int64_t period) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t j = i % period;
  y[i] = fmaf(x[i], __ldg(scale + j), __ldg(shift + j));
}

extern "C" int nes_affine_fwd(const float* x, const float* scale, const float* shift, float* y, int64_t n, int64_t period,
                              nes_stream_t stream) {
  NES_REQUIRE(n >= 0 && period > 0, NES_ERR_BAD_ARG, "affine_fwd: bad extent");
  if (n == 0) return NES_OK;
  NES_REQUIRE(x && scale && shift && y, NES_ERR_BAD_ARG, "affine_fwd: null pointer");
  NES_REQUIRE(ceil_div<int64_t>(n, 256) <= INT32_MAX, NES_ERR_UNSUPPORTED, "affine_fwd: too large");
  affine_kernel<<<(unsigned)ceil_div<int64_t>(n, 256), 256, 0, as_stream(stream)>>>(x, scale, shift, y, n, period);
  return check_launch("affine_fwd");
}

extern "C" int64_t nes_synthetic_linear_fwd_scratch_bytes(int64_t D, int64_t R, int64_t out) {
  return D * R * out * (int64_t)sizeof(float);
}

extern "C" int nes_synthetic_linear_fwd(const float* x, const float* weight, const float* bias,
                                        const float* eps, const float* bias_noise,
                                        const int8_t* fin, const int8_t* fout, float* y,
                                        int64_t D, int64_t R, int64_t in, int64_t out, int antithetic,
                                        void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0 && in >= 0 && out >= 0, NES_ERR_BAD_ARG, "synthetic_linear_fwd: negative extent");
  if (D == 0 || R == 0 || out == 0) return NES_OK;
  NES_REQUIRE(x && weight && eps && y, NES_ERR_BAD_ARG, "synthetic_linear_fwd: null pointer");
  NES_REQUIRE(scratch && scratch_bytes >= nes_synthetic_linear_fwd_scratch_bytes(D, R, out) && aligned16(scratch),
              NES_ERR_SCRATCH, "synthetic_linear_fwd: scratch needs %lld bytes, 16-byte aligned",
              (long long)nes_synthetic_linear_fwd_scratch_bytes(D, R, out));
  cudaStream_t st = as_stream(stream);
  const int64_t B = D * R;
  float* p = static_cast<float*>(scratch);
  BiasEpi none; none.bias = nullptr;
  int rc;
  if (fin) {
    FlipKLoader g; g.src = x; g.ld = in; g.rows = B; g.K = int(in); g.flips = fin; g.D = D;
    rc = launch_linear(g, eps, none, p, B, out, in, st, "synthetic_linear_fwd(noise)");
  } else {
    rc = launch_linear(rows_loader(x, in, B, int(in)), eps, none, p, B, out, in, st, "synthetic_linear_fwd(noise)");
  }
  if (rc != NES_OK) return rc;
  FlipEpi epi;
  epi.bias = bias; epi.p = p; epi.fout = fout; epi.bias_noise = bias_noise;
  epi.D = D; epi.R = R; epi.N = int(out); epi.antithetic = antithetic;
  return launch_linear(rows_loader(x, in, B, int(in)), weight, epi, y, B, out, in, st, "synthetic_linear_fwd(base)");
}
