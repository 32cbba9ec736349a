// Fitness-weighted noise reductions that form the weight update.
#include "common.cuh"

namespace nes {

// ---- sum_d w[d] * noise[d, :] : dense per-member noise ----------------------------------
//
// Streams the (D, n) noise once (HBM-bound).  A thread owns one 128-bit column group and walks
// a slice of the members with eight independent evict-first loads in flight.  The member
// range is split over blockIdx.y so that the grid fills the machine with an even number of
// waves; each split writes an fp32 partial row to scratch and a second kernel adds the
// partials in split order (deterministic) together with the l1 / l2 terms.
constexpr int UPD_THREADS = 256;
constexpr int UPD_BLOCKS_PER_SM = 4;
constexpr int UPD_MAX_SPLITS = 16;

// SUB: the tensors hold parameter + noise ("direct" storage); the parameter row `sub` is taken out of every
// member's row before it is weighted, so the sum never carries (sum_d w_d) * parameter around.
template <bool VEC, bool SUB>
__global__ void __launch_bounds__(UPD_THREADS, UPD_BLOCKS_PER_SM) weighted_noise_sum_kernel(
    const float* __restrict__ noise, const float* __restrict__ w, const float* __restrict__ sub,
    float* __restrict__ out, int64_t D, int64_t n, int64_t d_per_split, int64_t ld) {
  const int64_t d0 = blockIdx.y * d_per_split;
  const int64_t d1 = (d0 + d_per_split < D) ? d0 + d_per_split : D;
  float* dst = out + blockIdx.y * n;
  if (VEC) {
    const int64_t i4 = int64_t(blockIdx.x) * UPD_THREADS + threadIdx.x;
    if (i4 * 4 >= n) return;
    const float4* src = reinterpret_cast<const float4*>(noise) + i4;
    const int64_t stride = ld / 4;                  // row pitch of the noise in 128-bit units (ld == n unless a column block)
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 pv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (SUB) pv = __ldg(reinterpret_cast<const float4*>(sub) + i4);
    int64_t d = d0;
    for (; d + 8 <= d1; d += 8) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcs(src + (d + u) * stride);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float wd = __ldg(w + d + u);
        if (SUB) { v[u].x -= pv.x; v[u].y -= pv.y; v[u].z -= pv.z; v[u].w -= pv.w; }
        acc.x = fmaf(wd, v[u].x, acc.x); acc.y = fmaf(wd, v[u].y, acc.y);
        acc.z = fmaf(wd, v[u].z, acc.z); acc.w = fmaf(wd, v[u].w, acc.w);
      }
    }
    for (; d < d1; ++d) {
      float4 v = __ldcs(src + d * stride);
      const float wd = __ldg(w + d);
      if (SUB) { v.x -= pv.x; v.y -= pv.y; v.z -= pv.z; v.w -= pv.w; }
      acc.x = fmaf(wd, v.x, acc.x); acc.y = fmaf(wd, v.y, acc.y);
      acc.z = fmaf(wd, v.z, acc.z); acc.w = fmaf(wd, v.w, acc.w);
    }
    reinterpret_cast<float4*>(dst)[i4] = acc;
  } else {
    const int64_t i = int64_t(blockIdx.x) * UPD_THREADS + threadIdx.x;
    if (i >= n) return;
    float acc = 0.f;
    const float pv = SUB ? __ldg(sub + i) : 0.f;
    for (int64_t d = d0; d < d1; ++d) acc = fmaf(__ldg(w + d), __ldcs(noise + d * ld + i) - pv, acc);
    dst[i] = acc;
  }
}

// grad = sum_s partial[s] (+ l1 sign(W) + l2 W); splits == 0 means "grad already holds the sum"
__global__ void finish_update_kernel(const float* __restrict__ partial, int splits, const float* __restrict__ weight,
                                     float* __restrict__ grad, int64_t n, float l1, float l2) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = splits ? 0.f : grad[i];
  for (int s = 0; s < splits; ++s) acc += partial[s * n + i];
  if (weight) {
    const float wv = weight[i];
    if (l1 != 0.f) acc += l1 * ((wv > 0.f) - (wv < 0.f));
    if (l2 != 0.f) acc += l2 * wv;
  }
  grad[i] = acc;
}

struct UpdatePlan { int splits; int64_t d_per_split; int64_t bx; bool vec; };

static UpdatePlan plan_update(int64_t D, int64_t n, bool vec) {
  UpdatePlan p;
  p.vec = vec;
  const int64_t cols = vec ? n / 4 : n;
  p.bx = ceil_div<int64_t>(cols, UPD_THREADS);
  const int64_t slots = int64_t(sm_count()) * UPD_BLOCKS_PER_SM;
  int best = 1;
  if (p.bx < 4 * slots) {
    // smallest split count that gives at least two waves with a last wave >= 95 % full;
    // failing that, the candidate with the fullest last wave
    const int64_t cap = D / 8;
    const int max_s = int(cap > UPD_MAX_SPLITS ? UPD_MAX_SPLITS : (cap > 1 ? cap : 1));
    double best_score = -1.0;
    for (int s = 1; s <= max_s; ++s) {
      const int64_t items = p.bx * s;
      const double eff = double(items) / double(ceil_div(items, slots) * slots);
      const bool enough = items >= 2 * slots;
      if (enough && eff >= 0.95) { best = s; break; }
      const double score = (enough ? 1.0 : 0.0) + eff;
      if (score > best_score) { best_score = score; best = s; }
    }
  }
  p.splits = best;
  p.d_per_split = ceil_div<int64_t>(D, best);
  p.splits = int(ceil_div<int64_t>(D, p.d_per_split));
  return p;
}

// ---- shared noise + permutations ---------------------------------------------------------

// out-only: G[k, s] += w_d for s = pout[d,k] < out_sp;  in-only: H[j, pin[d,j]] += w_d
__global__ void permutation_histogram_kernel(const int16_t* __restrict__ perm, const float* __restrict__ w,
                                             float* __restrict__ hist, int64_t D, int cols, int hist_cols,
                                             int limit) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= D * cols) return;
  const int64_t d = e / cols;
  const int c = int(e - d * cols);
  const int s = perm[e];
  if (s < limit) atomicAdd(hist + size_t(c) * hist_cols + s, __ldg(w + d));
}

// grad[k,m,t] = sum_s G[k,s] * eps[s,m,t]     (out-only; eps has `in` input channels)
__global__ void grad_from_out_hist_kernel(const float* __restrict__ G, const float* __restrict__ eps,
                                          float* __restrict__ grad, int out, int out_sp, int64_t inner) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;   // over inner = in*ksz
  const int k = blockIdx.y;
  if (e >= inner) return;
  const float* g = G + size_t(k) * out_sp;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int s = 0;
  for (; s + 4 <= out_sp; s += 4) {
    a0 = fmaf(__ldg(g + s), __ldg(eps + (s + 0) * inner + e), a0);
    a1 = fmaf(__ldg(g + s + 1), __ldg(eps + (s + 1) * inner + e), a1);
    a2 = fmaf(__ldg(g + s + 2), __ldg(eps + (s + 2) * inner + e), a2);
    a3 = fmaf(__ldg(g + s + 3), __ldg(eps + (s + 3) * inner + e), a3);
  }
  for (; s < out_sp; ++s) a0 = fmaf(__ldg(g + s), __ldg(eps + s * inner + e), a0);
  grad[size_t(k) * inner + e] = (a0 + a1) + (a2 + a3);
}

// Output-permuted update in ONE launch (weight gradient, bias gradient, l1 / l2 terms):
//   grad[k, e]  = sum_s G[k,s] * eps[s, e] (+ l1 sign(W) + l2 W),   G[k,s] = sum_d w_d [pout[d,k] == s, s < out_sp]
//   bias_grad[k] = sum_d w_d * beta[d,k]
// Blocks 0 .. gblocks-1 own PU_ROWS output rows each.  The rows' slice of G is built in shared memory with
// shared-memory atomics straight from the permutation table (no histogram in global memory, nothing to clear;
// a thread first loads the eight entries of a member, then adds them).  The product is latency-bound (every
// block reads all of eps from L2), so the noise rows are dealt round-robin to PU_SGROUPS thread groups that
// each walk their rows with PU_UNROLL 128-bit loads in flight per thread over 256 columns at a time; the
// groups' partial sums meet in shared memory.  The remaining blocks own 32 columns of the bias gradient each.
constexpr int PU_THREADS = 512, PU_SGROUPS = 8, PU_COLS = 256, PU_UNROLL = 8;

// PU_ROWS = 8 output rows per block, or 4 when eight would leave most of the SMs without a block
template <int PU_ROWS>
__global__ void __launch_bounds__(PU_THREADS) permuted_update_out_kernel(
    const float* __restrict__ eps, const float* __restrict__ w, const int16_t* __restrict__ pout,
    const float* __restrict__ weight, const float* __restrict__ beta, float* __restrict__ grad,
    float* __restrict__ bias_grad, int64_t D, int out, int out_sp, int64_t inner, int gblocks, float l1, float l2,
    int vec_eps, int vec_pout) {
  extern __shared__ __align__(16) float pu_smem[];
  const int t = threadIdx.x;
  if (int(blockIdx.x) >= gblocks) {
    // ---- bias gradient: 32 columns x 16 member lanes, the lanes' sums added in lane order
    const int c = (int(blockIdx.x) - gblocks) * 32 + (t & 31);
    const int lane_d = t >> 5;
    float acc = 0.f;
    if (c < out) {
#pragma unroll 8
      for (int64_t d = lane_d; d < D; d += PU_THREADS / 32) acc = fmaf(__ldg(w + d), __ldg(beta + d * out + c), acc);
    }
    pu_smem[t] = acc;
    __syncthreads();
    if (t < 32 && c < out) {
      float s = 0.f;
#pragma unroll
      for (int u = 0; u < PU_THREADS / 32; ++u) s += pu_smem[u * 32 + t];
      bias_grad[c] = s;
    }
    return;
  }
  float* Gs = pu_smem;                                            // [out_sp][PU_ROWS]
  float* red = pu_smem + size_t(out_sp) * PU_ROWS;                // [PU_SGROUPS][PU_ROWS][PU_COLS]
  const int k0 = blockIdx.x * PU_ROWS;
  for (int i = t; i < out_sp * PU_ROWS; i += PU_THREADS) Gs[i] = 0.f;
  __syncthreads();
  if (vec_pout && k0 + PU_ROWS <= out) {
    for (int64_t d = t; d < D; d += PU_THREADS) {
      uint32_t q[PU_ROWS / 2];
      if (PU_ROWS == 8) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(pout + d * out + k0));
        q[0] = v.x; q[1] = v.y; q[PU_ROWS / 2 - 2] = v.z; q[PU_ROWS / 2 - 1] = v.w;
      } else {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(pout + d * out + k0));
        q[0] = v.x; q[1] = v.y;
      }
      const float wd = __ldg(w + d);
#pragma unroll
      for (int u = 0; u < PU_ROWS / 2; ++u) {
        const int s0 = int(q[u] & 0xFFFFu), s1 = int(q[u] >> 16);
        if (s0 < out_sp) atomicAdd(&Gs[s0 * PU_ROWS + 2 * u], wd);
        if (s1 < out_sp) atomicAdd(&Gs[s1 * PU_ROWS + 2 * u + 1], wd);
      }
    }
  } else {
    for (int64_t i = t; i < D * PU_ROWS; i += PU_THREADS) {
      const int64_t d = i / PU_ROWS;
      const int kk = int(i - d * PU_ROWS);
      if (k0 + kk < out) {
        const int s = int(uint16_t(pout[d * out + k0 + kk]));
        if (s < out_sp) atomicAdd(&Gs[s * PU_ROWS + kk], __ldg(w + d));
      }
    }
  }
  __syncthreads();
  const int cg = t % (PU_COLS / 4), sg = t / (PU_COLS / 4);       // four columns and one group of noise rows per thread
  for (int64_t c0 = 0; c0 < inner; c0 += PU_COLS) {
    const int64_t e = c0 + 4 * cg;
    float a[PU_ROWS][4];
#pragma unroll
    for (int u = 0; u < PU_ROWS; ++u) { a[u][0] = a[u][1] = a[u][2] = a[u][3] = 0.f; }
    if (e < inner) {
      for (int sb = sg; sb < out_sp; sb += PU_SGROUPS * PU_UNROLL) {
        float4 ev[PU_UNROLL];
#pragma unroll
        for (int i = 0; i < PU_UNROLL; ++i) {
          const int s = sb + i * PU_SGROUPS;
          ev[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (s < out_sp) {
            const float* src = eps + int64_t(s) * inner + e;
            if (vec_eps) {
              ev[i] = __ldg(reinterpret_cast<const float4*>(src));
            } else {
              ev[i].x = __ldg(src);
              if (e + 1 < inner) ev[i].y = __ldg(src + 1);
              if (e + 2 < inner) ev[i].z = __ldg(src + 2);
              if (e + 3 < inner) ev[i].w = __ldg(src + 3);
            }
          }
        }
#pragma unroll
        for (int i = 0; i < PU_UNROLL; ++i) {
          const int s = sb + i * PU_SGROUPS;
          if (s < out_sp) {
            float g[PU_ROWS];
#pragma unroll
            for (int u4 = 0; u4 < PU_ROWS; u4 += 4) {
              const float4 gv = *reinterpret_cast<const float4*>(Gs + s * PU_ROWS + u4);
              g[u4] = gv.x; g[u4 + 1] = gv.y; g[u4 + 2] = gv.z; g[u4 + 3] = gv.w;
            }
#pragma unroll
            for (int u = 0; u < PU_ROWS; ++u) {
              a[u][0] = fmaf(g[u], ev[i].x, a[u][0]); a[u][1] = fmaf(g[u], ev[i].y, a[u][1]);
              a[u][2] = fmaf(g[u], ev[i].z, a[u][2]); a[u][3] = fmaf(g[u], ev[i].w, a[u][3]);
            }
          }
        }
      }
    }
    __syncthreads();                                              // previous pass has finished reading red
#pragma unroll
    for (int u = 0; u < PU_ROWS; ++u)
      *reinterpret_cast<float4*>(red + (size_t(sg) * PU_ROWS + u) * PU_COLS + 4 * cg) = make_float4(a[u][0], a[u][1], a[u][2], a[u][3]);
    __syncthreads();
    for (int i = t; i < PU_ROWS * PU_COLS; i += PU_THREADS) {
      const int u = i / PU_COLS, col = i - u * PU_COLS;
      if (k0 + u >= out || c0 + col >= inner) continue;
      float v = 0.f;
#pragma unroll
      for (int g = 0; g < PU_SGROUPS; ++g) v += red[(size_t(g) * PU_ROWS + u) * PU_COLS + col];
      const int64_t o = int64_t(k0 + u) * inner + c0 + col;
      if (weight) {
        const float wv = __ldg(weight + o);
        if (l1 != 0.f) v += l1 * ((wv > 0.f) - (wv < 0.f));
        if (l2 != 0.f) v += l2 * wv;
      }
      grad[o] = v;
    }
  }
}

// grad[k,m,t] = sum_j eps[k,j,t] * H[j,m]      (in-only)
// A block owns 128 columns m and HG_ROWS consecutive rows q = k*ksz + t; eps for those rows goes through
// shared memory in chunks of HG_CHUNK values of j, so every H element loaded feeds HG_ROWS products.
constexpr int HG_ROWS = 8, HG_CHUNK = 256;

__global__ void __launch_bounds__(128) grad_from_in_hist_kernel(const float* __restrict__ H, const float* __restrict__ eps,
                                                                float* __restrict__ grad, int in, int in_sp, int ksz, int rows) {
  __shared__ __align__(16) float es[HG_CHUNK][HG_ROWS];
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  const int q0 = blockIdx.y * HG_ROWS;
  float a[HG_ROWS];
#pragma unroll
  for (int u = 0; u < HG_ROWS; ++u) a[u] = 0.f;
  for (int j0 = 0; j0 < in_sp; j0 += HG_CHUNK) {
    __syncthreads();
    for (int e = threadIdx.x; e < HG_CHUNK * HG_ROWS; e += blockDim.x) {
      const int jj = e / HG_ROWS, u = e - jj * HG_ROWS;
      const int q = q0 + u, j = j0 + jj;
      float v = 0.f;
      if (q < rows && j < in_sp) {
        const int k = q / ksz, t = q - k * ksz;
        v = __ldg(eps + (size_t(k) * in_sp + j) * ksz + t);
      }
      es[jj][u] = v;
    }
    __syncthreads();
    if (m < in) {
      const int lim = (in_sp - j0 < HG_CHUNK) ? in_sp - j0 : HG_CHUNK;
      const float* hp = H + size_t(j0) * in + m;
#pragma unroll 4
      for (int jj = 0; jj < lim; ++jj) {
        const float h = __ldg(hp + size_t(jj) * in);
        const float4 e0 = *reinterpret_cast<const float4*>(&es[jj][0]);
        const float4 e1 = *reinterpret_cast<const float4*>(&es[jj][4]);
        a[0] = fmaf(e0.x, h, a[0]); a[1] = fmaf(e0.y, h, a[1]); a[2] = fmaf(e0.z, h, a[2]); a[3] = fmaf(e0.w, h, a[3]);
        a[4] = fmaf(e1.x, h, a[4]); a[5] = fmaf(e1.y, h, a[5]); a[6] = fmaf(e1.z, h, a[6]); a[7] = fmaf(e1.w, h, a[7]);
      }
    }
  }
  if (m >= in) return;
#pragma unroll
  for (int u = 0; u < HG_ROWS; ++u) {
    const int q = q0 + u;
    if (q < rows) {
      const int k = q / ksz, t = q - k * ksz;
      grad[(size_t(k) * in + m) * ksz + t] = a[u];
    }
  }
}

// both: grad[k, pin[d,j], t] += w_d * eps[pout[d,k], j, t]
__global__ void grad_two_sided_kernel(const float* __restrict__ eps, const float* __restrict__ w,
                                      const int16_t* __restrict__ pin, const int16_t* __restrict__ pout,
                                      float* __restrict__ grad, int64_t D, int in, int out, int in_sp,
                                      int out_sp, int ksz) {
  const int64_t per_member = int64_t(out) * in_sp * ksz;
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= D * per_member) return;
  const int64_t d = e / per_member;
  int64_t r = e - d * per_member;
  const int k = int(r / (int64_t(in_sp) * ksz));
  r -= int64_t(k) * in_sp * ksz;
  const int j = int(r / ksz), t = int(r - int64_t(j) * ksz);
  const int so = pout[d * out + k];
  if (so >= out_sp) return;
  const int m = pin[d * in_sp + j];
  atomicAdd(grad + (size_t(k) * in + m) * ksz + t, __ldg(w + d) * __ldg(eps + (size_t(so) * in_sp + j) * ksz + t));
}

// sparse: grad[o, idx[d,o,t]] += w_d * val[d,o,t]
__global__ void grad_sparse_kernel(const int32_t* __restrict__ idx, const float* __restrict__ val,
                                   const float* __restrict__ w, float* __restrict__ grad, int64_t D,
                                   int64_t in, int64_t out, int k) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= D * out * k) return;
  const int64_t d = e / (out * k);
  const int64_t o = (e / k) % out;
  atomicAdd(grad + o * in + idx[e], __ldg(w + d) * __ldg(val + e));
}

// sign-flip sampling: grad[k,m,t] = eps[k,m,t] * sum_d w_d * fout[d,k] * fin[d,m]  (missing side = +1)
__global__ void grad_synthetic_kernel(const float* __restrict__ eps, const float* __restrict__ w,
                                      const int8_t* __restrict__ fin, const int8_t* __restrict__ fout,
                                      float* __restrict__ grad, int64_t D, int in, int out, int ksz) {
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  const int k = blockIdx.y;
  if (m >= in) return;
  float a0 = 0.f, a1 = 0.f;
  int64_t d = 0;
  for (; d + 2 <= D; d += 2) {
    float f0 = __ldg(w + d), f1 = __ldg(w + d + 1);
    if (fout) { f0 *= float(fout[d * out + k]); f1 *= float(fout[(d + 1) * out + k]); }
    if (fin) { f0 *= float(fin[d * in + m]); f1 *= float(fin[(d + 1) * in + m]); }
    a0 += f0; a1 += f1;
  }
  for (; d < D; ++d) {
    float f0 = __ldg(w + d);
    if (fout) f0 *= float(fout[d * out + k]);
    if (fin) f0 *= float(fin[d * in + m]);
    a0 += f0;
  }
  const float fw = a0 + a1;
  const size_t base = (size_t(k) * in + m) * ksz;
  for (int t = 0; t < ksz; ++t) grad[base + t] = fw * __ldg(eps + base + t);
}

// One-sided sign flips: the flip weights do not depend on the other index, so they are summed once,
//   fw[c] = sum_d w_d * flips[d, c],
// (members split over blockIdx.y, fp32 atomics on the n sums) and the gradient is eps scaled by fw along that
// side: grad[k,m,t] = eps[k,m,t] * fw[k] (output flips) or * fw[m] (input flips).
__global__ void __launch_bounds__(128) flip_weight_sums_kernel(const float* __restrict__ w, const int8_t* __restrict__ flips,
                                                               float* __restrict__ fw, int64_t D, int n, int64_t d_per_block) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n) return;
  const int64_t d0 = blockIdx.y * d_per_block;
  const int64_t d1 = (d0 + d_per_block < D) ? d0 + d_per_block : D;
  float acc = 0.f;
#pragma unroll 8
  for (int64_t d = d0; d < d1; ++d) acc = fmaf(__ldg(w + d), float(flips[d * n + c]), acc);
  atomicAdd(fw + c, acc);
}

__global__ void grad_one_sided_flip_kernel(const float* __restrict__ eps, const float* __restrict__ fw, float* __restrict__ grad,
                                           int64_t total, int in, int ksz, int by_output) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int64_t km = e / ksz;                          // k * in + m
  const int idx = by_output ? int(km / in) : int(km % in);
  grad[e] = __ldg(eps + e) * __ldg(fw + idx);
}

static int finish(const float* partial, int splits, const float* weight, float* grad, int64_t n, float l1,
                  float l2, cudaStream_t st, const char* what) {
  if (splits == 0 && (weight == nullptr || (l1 == 0.f && l2 == 0.f))) return NES_OK;
  finish_update_kernel<<<(unsigned)ceil_div<int64_t>(n, 256), 256, 0, st>>>(partial, splits, weight, grad, n, l1, l2);
  return check_launch(what);
}

}  // namespace nes

using namespace nes;

// Workspace of the widest plan the reduction can choose for (D, n): the 128-bit form when the pointers allow
// it, the scalar form (four times as many column blocks, possibly another split count) when they do not.
static int64_t update_scratch_floats(int64_t D, int64_t n) {
  if (D <= 0 || n <= 0) return 0;
  int64_t need = 0;
  const UpdatePlan ps = plan_update(D, n, false);
  if (ps.splits > 1) need = int64_t(ps.splits) * n;
  if (n % 4 == 0) {
    const UpdatePlan pv = plan_update(D, n, true);
    if (pv.splits > 1 && int64_t(pv.splits) * n > need) need = int64_t(pv.splits) * n;
  }
  return need;
}

extern "C" int64_t nes_perturbed_update_scratch_bytes(int64_t D, int64_t n) {
  return update_scratch_floats(D, n) * (int64_t)sizeof(float);
}

static int run_perturbed_update(const float* noise, const float* w, const float* sub, const float* weight, float* grad,
                                int64_t D, int64_t n, float l1, float l2, void* scratch, int64_t scratch_bytes,
                                cudaStream_t st, int64_t ld = -1) {
  if (ld < 0) ld = n;
  NES_REQUIRE(D >= 0 && n >= 0 && ld >= n, NES_ERR_BAD_ARG, "perturbed_update: bad extent");
  if (n == 0) return NES_OK;
  NES_REQUIRE(grad && (D == 0 || (noise && w)), NES_ERR_BAD_ARG, "perturbed_update: null pointer");
  NES_REQUIRE((l1 == 0.f && l2 == 0.f) || weight, NES_ERR_BAD_ARG, "perturbed_update: l1/l2 given without weight");
  if (D == 0) {
    cudaMemsetAsync(grad, 0, n * sizeof(float), st);
    return finish(nullptr, 0, weight, grad, n, l1, l2, st, "perturbed_update(finish)");
  }
  const bool vec = (n % 4 == 0) && (ld % 4 == 0) && aligned16(noise) && aligned16(grad) && aligned16(scratch) && (!sub || aligned16(sub));
  const UpdatePlan p = plan_update(D, n, vec);
  NES_REQUIRE(p.bx <= INT32_MAX, NES_ERR_UNSUPPORTED, "perturbed_update: n too large");
  float* dst = grad;
  if (p.splits > 1) {
    NES_REQUIRE(scratch && scratch_bytes >= int64_t(p.splits) * n * (int64_t)sizeof(float), NES_ERR_SCRATCH,
                "perturbed_update: scratch needs %lld bytes", (long long)(int64_t(p.splits) * n * sizeof(float)));
    dst = static_cast<float*>(scratch);
  }
  dim3 grid((unsigned)p.bx, (unsigned)p.splits);
  if (sub) {
    if (vec) weighted_noise_sum_kernel<true, true><<<grid, UPD_THREADS, 0, st>>>(noise, w, sub, dst, D, n, p.d_per_split, ld);
    else weighted_noise_sum_kernel<false, true><<<grid, UPD_THREADS, 0, st>>>(noise, w, sub, dst, D, n, p.d_per_split, ld);
  } else {
    if (vec) weighted_noise_sum_kernel<true, false><<<grid, UPD_THREADS, 0, st>>>(noise, w, nullptr, dst, D, n, p.d_per_split, ld);
    else weighted_noise_sum_kernel<false, false><<<grid, UPD_THREADS, 0, st>>>(noise, w, nullptr, dst, D, n, p.d_per_split, ld);
  }
  int rc = check_launch("perturbed_update");
  if (rc != NES_OK) return rc;
  return finish(dst, p.splits > 1 ? p.splits : 0, weight, grad, n, l1, l2, st, "perturbed_update(finish)");
}

extern "C" int nes_perturbed_update(const float* noise, const float* w, const float* weight, float* grad,
                                    int64_t D, int64_t n, float l1, float l2,
                                    void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  return run_perturbed_update(noise, w, nullptr, weight, grad, D, n, l1, l2, scratch, scratch_bytes, as_stream(stream));
}

extern "C" int nes_perturbed_update_columns(const float* noise, const float* w, const float* weight, float* grad,
                                            int64_t D, int64_t n, int64_t ld, float l1, float l2,
                                            void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  return run_perturbed_update(noise, w, nullptr, weight, grad, D, n, l1, l2, scratch, scratch_bytes, as_stream(stream), ld);
}

extern "C" int nes_perturbed_update_direct(const float* stored, const float* w, const float* param, const float* weight,
                                           float* grad, int64_t D, int64_t n, float l1, float l2,
                                           void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  NES_REQUIRE(param != nullptr || n == 0, NES_ERR_BAD_ARG, "perturbed_update_direct: null parameter");
  return run_perturbed_update(stored, w, param, weight, grad, D, n, l1, l2, scratch, scratch_bytes, as_stream(stream));
}

// ---- the same reduction for callers that cannot supply a workspace -------------------------
//
// Built-in workspace for nes_perturbed_update_noalloc: NES_NOALLOC_SCRATCH_FLOATS fp32 values
// (16 MiB) that every GPU which loads this library keeps until the process exits.  In host code
// the array's name is only a stand-in for the symbol; the device address is looked up once per
// device and handed to the kernels as an ordinary pointer.
static __device__ __align__(256) float g_builtin_update_scratch[NES_NOALLOC_SCRATCH_FLOATS];

static int builtin_update_scratch(float** out) {
  static float* address_on_device[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "perturbed_update_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  NES_REQUIRE(dev >= 0 && dev < 64, NES_ERR_UNSUPPORTED, "perturbed_update_noalloc: device index %d out of range", dev);
  if (address_on_device[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_builtin_update_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(NES_ERR_LAUNCH, "perturbed_update_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    address_on_device[dev] = p;
  }
  *out = address_on_device[dev];
  return NES_OK;
}

extern "C" int nes_perturbed_update_noalloc(const float* noise, const float* w, const float* weight, float* grad,
                                            int64_t D, int64_t n, float l1, float l2, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && n >= 0, NES_ERR_BAD_ARG, "perturbed_update_noalloc: negative extent");
  if (n == 0) return NES_OK;
  // the workspace of whichever plan (128-bit or scalar columns) the pointers' alignment will select
  const int64_t need_floats = update_scratch_floats(D, n);
  NES_REQUIRE(need_floats <= (int64_t)NES_NOALLOC_SCRATCH_FLOATS, NES_ERR_UNSUPPORTED,
              "perturbed_update_noalloc: D=%lld, n=%lld needs %lld floats of workspace but the built-in one holds %lld; "
              "use nes_perturbed_update with a caller-owned scratch buffer",
              (long long)D, (long long)n, (long long)need_floats, (long long)NES_NOALLOC_SCRATCH_FLOATS);
  float* ws = nullptr;
  if (need_floats > 0) {
    int rc = builtin_update_scratch(&ws);
    if (rc != NES_OK) return rc;
  }
  return nes_perturbed_update(noise, w, weight, grad, D, n, l1, l2, ws,
                              (int64_t)NES_NOALLOC_SCRATCH_FLOATS * (int64_t)sizeof(float), stream);
}

extern "C" int64_t nes_permuted_update_scratch_bytes(int in, int out, int in_sp, int out_sp) {
  const int64_t g = int64_t(out) * out_sp, h = int64_t(in_sp) * in;
  return (g > h ? g : h) * (int64_t)sizeof(float);
}

extern "C" int nes_permuted_update(const float* eps, const float* w, const int16_t* pin, const int16_t* pout,
                                   const float* weight, float* grad, float* perm_weights_out,
                                   int64_t D, int in, int out, int in_sp, int out_sp, int ksize,
                                   float l1, float l2, void* scratch, int64_t scratch_bytes,
                                   nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && in > 0 && out > 0 && in_sp > 0 && out_sp > 0 && ksize > 0, NES_ERR_BAD_ARG,
              "permuted_update: bad extent");
  NES_REQUIRE(eps && grad && (D == 0 || w) && (pin || pout), NES_ERR_BAD_ARG, "permuted_update: null pointer");
  NES_REQUIRE((l1 == 0.f && l2 == 0.f) || weight, NES_ERR_BAD_ARG, "permuted_update: l1/l2 given without weight");
  NES_REQUIRE(out_sp <= out && (pin || in_sp == in), NES_ERR_BAD_ARG, "permuted_update: sparsity exceeds degree");
  NES_REQUIRE(out <= 65535 && int64_t(out) * ksize <= 65535, NES_ERR_UNSUPPORTED, "permuted_update: out*ksize > 65535");
  cudaStream_t st = as_stream(stream);
  const int64_t n = int64_t(out) * in * ksize;
  int rc;
  if (pin && pout) {
    cudaMemsetAsync(grad, 0, n * sizeof(float), st);
    const int64_t total = D * out * in_sp * ksize;
    if (total > 0) {
      NES_REQUIRE(ceil_div<int64_t>(total, 256) <= INT32_MAX, NES_ERR_UNSUPPORTED, "permuted_update: two-sided problem too large");
      grad_two_sided_kernel<<<(unsigned)ceil_div<int64_t>(total, 256), 256, 0, st>>>(eps, w, pin, pout, grad, D, in, out, in_sp, out_sp, ksize);
      rc = check_launch("permuted_update(two-sided)");
      if (rc != NES_OK) return rc;
    }
    return finish(nullptr, 0, weight, grad, n, l1, l2, st, "permuted_update(finish)");
  }
  NES_REQUIRE(scratch && scratch_bytes >= nes_permuted_update_scratch_bytes(in, out, in_sp, out_sp), NES_ERR_SCRATCH,
              "permuted_update: scratch needs %lld bytes", (long long)nes_permuted_update_scratch_bytes(in, out, in_sp, out_sp));
  float* hist = static_cast<float*>(scratch);
  if (pout) {
    const int64_t hn = int64_t(out) * out_sp;
    cudaMemsetAsync(hist, 0, hn * sizeof(float), st);
    if (D > 0) {
      permutation_histogram_kernel<<<(unsigned)ceil_div<int64_t>(D * out, 256), 256, 0, st>>>(pout, w, hist, D, out, out_sp, out_sp);
      rc = check_launch("permuted_update(histogram)");
      if (rc != NES_OK) return rc;
    }
    const int64_t inner = int64_t(in) * ksize;
    dim3 grid((unsigned)ceil_div<int64_t>(inner, 256), (unsigned)out);
    grad_from_out_hist_kernel<<<grid, 256, 0, st>>>(hist, eps, grad, out, out_sp, inner);
    rc = check_launch("permuted_update(grad)");
    if (rc != NES_OK) return rc;
    if (perm_weights_out) cudaMemcpyAsync(perm_weights_out, hist, hn * sizeof(float), cudaMemcpyDeviceToDevice, st);
  } else {
    const int64_t hn = int64_t(in_sp) * in;
    cudaMemsetAsync(hist, 0, hn * sizeof(float), st);
    if (D > 0) {
      permutation_histogram_kernel<<<(unsigned)ceil_div<int64_t>(D * in_sp, 256), 256, 0, st>>>(pin, w, hist, D, in_sp, in, in);
      rc = check_launch("permuted_update(histogram)");
      if (rc != NES_OK) return rc;
    }
    dim3 grid((unsigned)ceil_div(in, 128), (unsigned)ceil_div(out * ksize, HG_ROWS));
    grad_from_in_hist_kernel<<<grid, 128, 0, st>>>(hist, eps, grad, in, in_sp, ksize, out * ksize);
    rc = check_launch("permuted_update(grad)");
    if (rc != NES_OK) return rc;
    if (perm_weights_out) cudaMemcpyAsync(perm_weights_out, hist, hn * sizeof(float), cudaMemcpyDeviceToDevice, st);
  }
  return finish(nullptr, 0, weight, grad, n, l1, l2, st, "permuted_update(finish)");
}

extern "C" int nes_permuted_update_out(const float* eps, const float* w, const int16_t* pout, const float* weight,
                                       const float* bias_noise, float* grad, float* bias_grad,
                                       int64_t D, int in, int out, int out_sp, int ksize, float l1, float l2,
                                       nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && in > 0 && out > 0 && out_sp > 0 && ksize > 0 && out_sp <= out, NES_ERR_BAD_ARG,
              "permuted_update_out: bad extent");
  NES_REQUIRE(eps && grad && pout && (D == 0 || w), NES_ERR_BAD_ARG, "permuted_update_out: null pointer");
  NES_REQUIRE((l1 == 0.f && l2 == 0.f) || weight, NES_ERR_BAD_ARG, "permuted_update_out: l1/l2 given without weight");
  NES_REQUIRE((bias_noise == nullptr) == (bias_grad == nullptr), NES_ERR_BAD_ARG,
              "permuted_update_out: bias_noise and bias_grad go together");
  const int rows = (ceil_div(out, 8) * 2 <= sm_count()) ? 4 : 8;       // more, smaller blocks while the grid is far below the SM count
  const size_t smem = (size_t(out_sp) * rows + size_t(PU_SGROUPS) * rows * PU_COLS) * sizeof(float);
  NES_REQUIRE(smem <= 200 * 1024, NES_ERR_UNSUPPORTED, "permuted_update_out: out_sp=%d needs %zu B of shared memory", out_sp, smem);
  const size_t smem_all = smem;
  auto kern = rows == 4 ? permuted_update_out_kernel<4> : permuted_update_out_kernel<8>;
  if (smem_all > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_all);
    if (e != cudaSuccess) return fail(NES_ERR_UNSUPPORTED, "permuted_update_out: %zu B of shared memory refused", smem_all);
  }
  const int gblocks = ceil_div(out, rows);
  const int bblocks = bias_grad ? ceil_div(out, 32) : 0;
  kern<<<gblocks + bblocks, PU_THREADS, smem_all, as_stream(stream)>>>(
      eps, w, pout, (l1 != 0.f || l2 != 0.f) ? weight : nullptr, bias_noise, grad, bias_grad, D, out, out_sp,
      int64_t(in) * ksize, gblocks, l1, l2,
      ((int64_t(in) * ksize) % 4 == 0 && aligned16(eps)) ? 1 : 0, (out % 8 == 0 && aligned16(pout)) ? 1 : 0);
  return check_launch("permuted_update_out");
}

extern "C" int nes_sparse_perturbed_update(const int32_t* idx, const float* val, const float* w,
                                           const float* weight, float* grad, int64_t D, int64_t in,
                                           int64_t out, int k, float l1, float l2, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && in > 0 && out > 0 && k >= 0, NES_ERR_BAD_ARG, "sparse_perturbed_update: bad extent");
  NES_REQUIRE(grad && (D * k == 0 || (idx && val && w)), NES_ERR_BAD_ARG, "sparse_perturbed_update: null pointer");
  NES_REQUIRE((l1 == 0.f && l2 == 0.f) || weight, NES_ERR_BAD_ARG, "sparse_perturbed_update: l1/l2 given without weight");
  cudaStream_t st = as_stream(stream);
  cudaMemsetAsync(grad, 0, out * in * sizeof(float), st);
  const int64_t total = D * out * k;
  if (total > 0) {
    NES_REQUIRE(ceil_div<int64_t>(total, 256) <= INT32_MAX, NES_ERR_UNSUPPORTED, "sparse_perturbed_update: too large");
    grad_sparse_kernel<<<(unsigned)ceil_div<int64_t>(total, 256), 256, 0, st>>>(idx, val, w, grad, D, in, out, k);
    int rc = check_launch("sparse_perturbed_update");
    if (rc != NES_OK) return rc;
  }
  return finish(nullptr, 0, weight, grad, out * in, l1, l2, st, "sparse_perturbed_update(finish)");
}

extern "C" int64_t nes_synthetic_update_scratch_bytes(int in, int out) { return int64_t(in > out ? in : out) * 4; }

extern "C" int nes_synthetic_update(const float* eps, const float* w, const int8_t* fin, const int8_t* fout,
                                    const float* weight, float* grad, int64_t D, int in, int out, int ksize,
                                    float l1, float l2, void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && in > 0 && out > 0 && ksize > 0, NES_ERR_BAD_ARG, "synthetic_update: bad extent");
  NES_REQUIRE(eps && grad && (D == 0 || w) && (fin || fout), NES_ERR_BAD_ARG, "synthetic_update: null pointer");
  NES_REQUIRE((l1 == 0.f && l2 == 0.f) || weight, NES_ERR_BAD_ARG, "synthetic_update: l1/l2 given without weight");
  NES_REQUIRE(out <= 65535, NES_ERR_UNSUPPORTED, "synthetic_update: out > 65535");
  cudaStream_t st = as_stream(stream);
  int rc;
  const int64_t total = int64_t(out) * in * ksize;
  if ((fin == nullptr) != (fout == nullptr) && scratch && scratch_bytes >= int64_t(in > out ? in : out) * 4) {
    // one flipped side: n flip-weight sums, then a scaling of eps
    const int n = fout ? out : in;
    float* fw = static_cast<float*>(scratch);
    cudaMemsetAsync(fw, 0, size_t(n) * sizeof(float), st);
    if (D > 0) {
      const int slices = int(D < 64 ? 1 : (D / 32 < 64 ? D / 32 : 64));
      const int64_t per = ceil_div<int64_t>(D, slices);
      dim3 sgrid((unsigned)ceil_div(n, 128), (unsigned)ceil_div<int64_t>(D, per));
      flip_weight_sums_kernel<<<sgrid, 128, 0, st>>>(w, fout ? fout : fin, fw, D, n, per);
      if ((rc = check_launch("synthetic_update(flip sums)")) != NES_OK) return rc;
    }
    grad_one_sided_flip_kernel<<<(unsigned)ceil_div<int64_t>(total, 256), 256, 0, st>>>(eps, fw, grad, total, in, ksize, fout ? 1 : 0);
    if ((rc = check_launch("synthetic_update(scale)")) != NES_OK) return rc;
    return finish(nullptr, 0, weight, grad, total, l1, l2, st, "synthetic_update(finish)");
  }
  dim3 grid((unsigned)ceil_div(in, 128), (unsigned)out);
  grad_synthetic_kernel<<<grid, 128, 0, st>>>(eps, w, fin, fout, grad, D, in, out, ksize);
  rc = check_launch("synthetic_update");
  if (rc != NES_OK) return rc;
  return finish(nullptr, 0, weight, grad, int64_t(out) * in * ksize, l1, l2, st, "synthetic_update(finish)");
}
