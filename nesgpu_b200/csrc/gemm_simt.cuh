// fp32 CUDA-core GEMM skeleton shared by the exact-fp32 layer kernels.
//
// One thread block computes a 128x128 (or 128x64) tile of C = A . B^T with K stepped by 16, 256 threads,
// an 8x8 micro-tile per thread (two 4-wide groups 64 apart in each direction so that the
// shared-memory reads are conflict-free 128-bit loads), double-buffered shared memory with
// the next tile's global loads issued before the current tile's math.
//
// A "problem" type supplies: how a tile of A and of B is fetched (registers) and stored
// (shared memory, always as [k][row]), and what happens to the accumulators.  That is where
// the layers differ: plain rows, rows gathered through a member's input permutation,
// im2col patches; plain weights or a member's effective filter W + s*E_d built on the fly;
// plain store or the permuted-output / bias-noise / antithetic-sign epilogue.
#pragma once
#include "common.cuh"

namespace nes {
namespace simt {

constexpr int BM = 128, BN = 128, BK = 16, NT = 256;
constexpr int LDS = 132;  // padded tile row (floats); keeps float4 alignment

struct Frag { float v[8]; };  // the 128*16/256 operand elements one thread stages per k-step

typedef float (*TilePtr)[LDS];

// ---- operand loaders -----------------------------------------------------------------

// Rows contiguous along K: src[row * ld + k].  Thread t covers rows t/4 and t/4+64, four
// consecutive k starting at (t%4)*4 (one 128-bit load each when `vec`).
struct RowsLoader {
  const float* src; int64_t ld; int64_t rows; int K; int vec;
  template <int ROWS>
  __device__ inline void fetch(int64_t row0, int k0, Frag& f) const {
    const int t = threadIdx.x;
    const int kq = k0 + (t & 3) * 4;
#pragma unroll
    for (int i = 0; i < ROWS / 64; ++i) {
      const int64_t row = row0 + (t >> 2) + 64 * i;
      float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row < rows) {
        const float* p = src + row * ld + kq;
        if (vec && kq + 3 < K) {
          val = __ldg(reinterpret_cast<const float4*>(p));
        } else {
          if (kq + 0 < K) val.x = __ldg(p + 0);
          if (kq + 1 < K) val.y = __ldg(p + 1);
          if (kq + 2 < K) val.z = __ldg(p + 2);
          if (kq + 3 < K) val.w = __ldg(p + 3);
        }
      }
      f.v[i * 4 + 0] = val.x; f.v[i * 4 + 1] = val.y; f.v[i * 4 + 2] = val.z; f.v[i * 4 + 3] = val.w;
    }
  }
  template <int ROWS>
  __device__ static inline void store(TilePtr T, const Frag& f) {
    const int t = threadIdx.x;
    const int kq = (t & 3) * 4;
#pragma unroll
    for (int i = 0; i < ROWS / 64; ++i) {
      const int r = (t >> 2) + 64 * i;
#pragma unroll
      for (int j = 0; j < 4; ++j) T[kq + j][r] = f.v[i * 4 + j];
    }
  }
};

// Element-wise mapping used by the gather / effective-weight loaders: thread t owns column
// k = t%16 of the k-step and rows t/16 + 16*i, i = 0..7.
template <int ROWS>
__device__ inline void store_elementwise(TilePtr T, const Frag& f) {
  const int t = threadIdx.x;
  const int k = t & 15;
#pragma unroll
  for (int i = 0; i < ROWS / 16; ++i) T[k][(t >> 4) + 16 * i] = f.v[i];
}

// Rows gathered along K through a per-member index table:
//   A[row, k] = src[row * ld + perm[(row % D) * K + k]]      (apply_input_permutation)
struct GatherKLoader {
  const float* src; int64_t ld; int64_t rows; int K; const int16_t* perm; int64_t D;
  template <int ROWS>
  __device__ inline void fetch(int64_t row0, int k0, Frag& f) const {
    const int t = threadIdx.x;
    const int k = k0 + (t & 15);
#pragma unroll
    for (int i = 0; i < ROWS / 16; ++i) {
      const int64_t row = row0 + (t >> 4) + 16 * i;
      float val = 0.f;
      if (row < rows && k < K) {
        const int idx = perm[(row % D) * K + k];
        val = __ldg(src + row * ld + idx);
      }
      f.v[i] = val;
    }
  }
  template <int ROWS>
  __device__ static inline void store(TilePtr T, const Frag& f) { store_elementwise<ROWS>(T, f); }
};

// Rows multiplied element-wise by a per-member sign vector:
//   A[row, k] = src[row * ld + k] * flips[(row % D) * K + k]      (sign-flip sampling, flips are +-1 int8)
struct FlipKLoader {
  const float* src; int64_t ld; int64_t rows; int K; const int8_t* flips; int64_t D;
  template <int ROWS>
  __device__ inline void fetch(int64_t row0, int k0, Frag& f) const {
    const int t = threadIdx.x;
    const int k = k0 + (t & 15);
#pragma unroll
    for (int i = 0; i < ROWS / 16; ++i) {
      const int64_t row = row0 + (t >> 4) + 16 * i;
      float val = 0.f;
      if (row < rows && k < K) val = __ldg(src + row * ld + k) * float(flips[(row % D) * K + k]);
      f.v[i] = val;
    }
  }
  template <int ROWS>
  __device__ static inline void store(TilePtr T, const Frag& f) { store_elementwise<ROWS>(T, f); }
};

// ---- the kernel ------------------------------------------------------------------------

template <class Prob>
__global__ void __launch_bounds__(NT) gemm_kernel(const Prob p) {
  __shared__ __align__(16) float As[2][BK][LDS];
  __shared__ __align__(16) float Bs[2][BK][LDS];
  typename Prob::Ctx ctx;
  p.init(ctx);
  const int K = p.k_extent();
  const int nk = ceil_div(K, BK);
  const int t = threadIdx.x;
  const int tm = Prob::MFAST ? (t & 15) : (t >> 4);
  const int tn = Prob::MFAST ? (t >> 4) : (t & 15);

  constexpr int NJ = Prob::NJ;   // n-groups of 4 per thread: 2 -> 128-wide tile, 1 -> 64-wide
  float acc[8][4 * NJ];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4 * NJ; ++j) acc[i][j] = 0.f;

  Frag fa, fb;
  p.fetchA(ctx, 0, fa);
  p.fetchB(ctx, 0, fb);
  p.storeA(As[0], fa);
  p.storeB(Bs[0], fb);
  __syncthreads();

  for (int kt = 0; kt < nk; ++kt) {
    const int cur = kt & 1;
    const bool more = (kt + 1 < nk);
    if (more) {
      p.fetchA(ctx, (kt + 1) * BK, fa);
      p.fetchB(ctx, (kt + 1) * BK, fb);
    }
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[cur][k][tm * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[cur][k][64 + tm * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[cur][k][tn * 4]);
      float4 b1 = b0;
      if (NJ == 2) b1 = *reinterpret_cast<const float4*>(&Bs[cur][k][64 + tn * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4 * NJ; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (more) {
      p.storeA(As[cur ^ 1], fa);
      p.storeB(Bs[cur ^ 1], fb);
    }
    __syncthreads();
  }
  p.epilogue(ctx, acc, tm, tn);
}

// local (within-tile) row / column of accumulator index i or j
__device__ inline int micro_index(int tgroup, int i) { return (i < 4) ? (tgroup * 4 + i) : (64 + tgroup * 4 + i - 4); }

}  // namespace simt
}  // namespace nes
