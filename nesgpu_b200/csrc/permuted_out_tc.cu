// Output-permuted PermutedLinear forward as ONE tensor-core kernel (sm_100a).
//
//   y[b,k] = x[b].W[k] + bias[k] + s(r) * ( p[b, pout[d,k]] + beta[d,k] ),   p[b,s] = x[b].eps[s]
//
// with b = r*D + d (modules/base.py:487-508 with permute_inputs off).  Consecutive batch rows belong to
// different members, so no tile of rows shares a permutation: the layer is evaluated as the stacked
// product x.[W; eps]^T and the per-row gather p[b, pout[d,k]] happens in the epilogue, on accumulators
// that never leave the chip.
//
// Work split.  A thread-block cluster of S blocks owns one tile of 128 batch rows; block j of the
// cluster owns the base columns [j*NB, (j+1)*NB) and the noise columns [j*NP, (j+1)*NP), i.e. it
// multiplies the row tile by the NB + NP stacked rows [W_j; eps_j] with ONE tcgen05.mma per K step
// (M = 128, N = NB + NP <= 256, K = 8, kind::tf32, fp32 accumulators in tensor memory).  After the K
// loop every block copies its noise accumulator (128 x NP) into shared memory and the blocks of the
// cluster exchange these slices through distributed shared memory: when the whole 128 x out_sp noise
// tile fits beside nothing else (the operand ring is idle by then), each block pushes its slice to its
// peers with one bulk copy per peer (cp.async.bulk shared::cta -> shared::cluster, completion counted
// on the receiver's mbarrier) and the gather p[row, pout[d,k]] runs on local shared memory; otherwise
// the gather reads single values from the owning block (ld.shared::cluster; about four cycles per
// value and SM, measured).  The block then adds base, bias, sign and beta and stores its NB columns of
// y.  Nothing but x, W, eps, pout, beta and y touches global memory.
//
// Operand path.  The fp32 tiles of x, W and eps arrive by TMA (128-byte swizzle) exactly as they lie in
// memory.  Four warps then split every tile in place: hi = tf32(a) overwrites the tile, lo = a - hi goes
// to a second tile of the same layout, and the MMA warp issues a_lo.b_hi + a_hi.b_lo + a_hi.b_hi
// (3xTF32, fp32-level accuracy; TERMS = 1 rounds in place and issues one product: plain TF32, for
// callers that state it).  No pre-pass, no scratch memory, one launch.
//
// Pipeline per block: warp 0 = TMA producer, warp 1 = MMA issuer (and owner of the tensor-memory
// allocation), warps 2-9 = operand splitters during the K loop and epilogue afterwards (two warps per
// tensor-memory lane quadrant, which take alternate 16-column chunks).  Stage hand-over
// by mbarriers: full (TMA bytes landed) -> split (hi/lo written, made visible to the async proxy) ->
// tcgen05.commit -> empty.  Every mbarrier wait is bounded; a wait that runs out records a code (see
// tc_ptx.cuh), the role stops issuing work and all threads still reach the two cluster barriers and the
// common exit where tensor memory is freed.  Every TMA load targets one block only.
#include <cuda.h>
#include "tc_ptx.cuh"

namespace nes {
namespace tc {

constexpr int PO_BM = 128;                 // batch rows per cluster
constexpr int PO_BK = 32;                  // fp32 K elements per stage = one 128-byte swizzle row
constexpr int PO_THREADS = 320;
constexpr int PO_WORKERS = PO_THREADS - 64;   // splitter / epilogue threads
constexpr int PO_A_BYTES = PO_BM * PO_BK * 4;
constexpr int PO_MIN_SMEM = 116 * 1024;    // more than half an SM's shared memory: one block per SM, so a block
                                           // that waits for its cluster never holds tensor memory a peer needs

struct PermOutParams {
  CUtensorMap map_x, map_w, map_eps;
  const float* bias; const float* beta; const int16_t* pout; float* y;
  long long B, D, R;
  int out, out_sp, K;
  int NB, NP;                               // base / noise columns per block (multiples of 16)
  int stages, tmem_cols, antithetic;
  unsigned int np_magic;                    // ceil(2^32 / NP): so / NP == umulhi(so, np_magic) for so < 2^24
  int vec_y, vec_pout, vec_beta, vec_bias;
  int local_gather;                         // 1: slices are pushed to the peers and the gather is local
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// All threads of all blocks of the cluster; release / acquire so that shared-memory writes made before the
// barrier are visible to the other blocks' distributed-shared-memory reads after it.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
// own shared memory -> the same place in a peer's shared memory; the peer's mbarrier counts the bytes
__device__ __forceinline__ void bulk_push(uint32_t remote_dst, uint32_t local_src, uint32_t bytes, uint32_t remote_bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(remote_dst), "r"(local_src), "r"(bytes), "r"(remote_bar)
      : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// asks the TMA unit to bring one box of a tiled tensor into L2 (no shared-memory destination, no barrier)
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Optional phase timestamps (build with -DNES_PO_TRACE): slot [block * 16 + phase] holds %globaltimer in ns.
#ifdef NES_PO_TRACE
__device__ long long g_po_trace[64 * 16];
__device__ __forceinline__ void po_trace(int phase) {
  const int blk = blockIdx.y * gridDim.x + blockIdx.x;
  if (blk < 64) {
    long long tns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tns));
    g_po_trace[blk * 16 + phase] = tns;
  }
}
#define PO_TRACE(cond, phase) do { if (cond) po_trace(phase); } while (0)
#else
#define PO_TRACE(cond, phase) do { } while (0)
#endif

template <int TERMS>
__global__ void __launch_bounds__(PO_THREADS, 1) permuted_linear_out_kernel(const __grid_constant__ PermOutParams p) {
  extern __shared__ unsigned char dyn_raw[];
  const unsigned int timeouts_at_start = timeouts_so_far();
  const uint32_t raw = smem_u32(dyn_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  unsigned char* tiles = dyn_raw + pad;
  const int NC = p.NB + p.NP;
  const int b_bytes = NC * PO_BK * 4;
  const int stage_bytes = (TERMS == 3 ? 2 : 1) * (PO_A_BYTES + b_bytes);
  // barriers sit behind the larger of the stage ring and the exchange area that reuses it
  const int pitch = p.NP + 4;                                  // floats per exchange row: 16-byte rows, rows 4 banks apart
  const int S = int(gridDim.x);
  const uint32_t slice_floats = uint32_t(PO_BM) * uint32_t(pitch);
  const size_t ring_bytes = size_t(p.stages) * stage_bytes;
  const size_t xchg_bytes = size_t(p.local_gather ? S : 1) * slice_floats * 4;
  const size_t body = ((ring_bytes > xchg_bytes ? ring_bytes : xchg_bytes) + 15) & ~size_t(15);
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + body);
  uint64_t* split = full + p.stages;
  uint64_t* empty = split + p.stages;
  uint64_t* accum = empty + p.stages;
  uint64_t* xbar = accum + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xbar + 1);
  float* xchg = reinterpret_cast<float*>(tiles);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t j = cluster_rank();                           // column slice of this block
  const long long m0 = (long long)blockIdx.y * PO_BM;
  const int nk = (p.K + PO_BK - 1) / PO_BK;
  float* my_slice = xchg + (p.local_gather ? size_t(j) * slice_floats : 0);
  PO_TRACE(threadIdx.x == 0, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&split[s], PO_WORKERS / 32); mbar_init(&empty[s], 1); }
    mbar_init(accum, 1);
    mbar_init(xbar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, uint32_t(p.tmem_cols));
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  PO_TRACE(threadIdx.x == 0, 1);

  // epilogue geometry of this thread (warps 2-9): accumulator row and the 16-column chunks it takes
  constexpr int PO_PRE = 2;                                    // chunks whose tables are preloaded into registers
  uint4 pre_so[PO_PRE][2];
  float4 pre_bn[PO_PRE][4], pre_bias[PO_PRE][4];
  const int q = warp & 3;
  const int row = q * 32 + lane;
  const int chunk0 = (warp - 2) >> 2;                          // 0 for warps 2-5, 1 for warps 6-9
  const long long gm = m0 + row;
  const int kbase = int(j) * p.NB;

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: the raw fp32 tiles of x, W_j and eps_j.  Once the ring is full, everything else this
      // block will read is requested into L2 (the ring holds only a few K steps, and a cold tile would cost an
      // HBM round trip each time a stage is refilled)
      for (int kt = 0; kt < nk; ++kt) {
        if (kt == p.stages) {
          for (int kp = p.stages; kp < nk; ++kp) {
            tma_prefetch_2d(&p.map_x, kp * PO_BK, int(m0));
            tma_prefetch_2d(&p.map_w, kp * PO_BK, int(j) * p.NB);
            tma_prefetch_2d(&p.map_eps, kp * PO_BK, int(j) * p.NP);
          }
        }
        const int s = kt % p.stages;
        const uint32_t ph = (kt / p.stages) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, 1)) break;
        unsigned char* st = tiles + size_t(s) * stage_bytes;
        unsigned char* bt = st + (TERMS == 3 ? 2 : 1) * PO_A_BYTES;
        mbar_expect_tx(&full[s], uint32_t(PO_A_BYTES + b_bytes));
        tma_load_2d(st, &p.map_x, &full[s], kt * PO_BK, int(m0));
        tma_load_2d(bt, &p.map_w, &full[s], kt * PO_BK, int(j) * p.NB);
        tma_load_2d(bt + size_t(p.NB) * PO_BK * 4, &p.map_eps, &full[s], kt * PO_BK, int(j) * p.NP);
        PO_TRACE(kt == 0, 2);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the whole warp runs this loop in converged control flow, one elected lane issues
    const uint32_t idesc = idesc_tf32(PO_BM, NC);
    bool ok = true;
    for (int kt = 0; kt < nk && ok; ++kt) {
      const int s = kt % p.stages;
      const uint32_t ph = (kt / p.stages) & 1;
      ok = warp_mbar_wait(&split[s], ph, 2);
      if (!ok) break;
      PO_TRACE(lane == 0 && kt == 0, 5);
      tc_fence_after();
      const uint32_t st = smem_u32(tiles + size_t(s) * stage_bytes);
      const uint64_t a_hi = smem_desc_sw128(st);
      const uint64_t a_lo = smem_desc_sw128(st + PO_A_BYTES);
      const uint32_t bt = st + (TERMS == 3 ? 2 : 1) * PO_A_BYTES;
      const uint64_t b_hi = smem_desc_sw128(bt);
      const uint64_t b_lo = smem_desc_sw128(bt + b_bytes);
#pragma unroll
      for (int k = 0; k < PO_BK / 8; ++k) {                   // 32 bytes (2 descriptor units) per K = 8
        const uint64_t adv = uint64_t(k * 2);
        const uint32_t first = (kt > 0 || k > 0) ? 1u : 0u;
        if (TERMS == 3) {
          warp_mma_tf32(tmem_base, a_lo + adv, b_hi + adv, idesc, first);
          warp_mma_tf32(tmem_base, a_hi + adv, b_lo + adv, idesc, 1u);
          warp_mma_tf32(tmem_base, a_hi + adv, b_hi + adv, idesc, 1u);
        } else {
          warp_mma_tf32(tmem_base, a_hi + adv, b_hi + adv, idesc, first);
        }
      }
      warp_mma_commit(&empty[s]);
    }
    warp_mma_commit(accum);
    PO_TRACE(lane == 0, 6);
  } else {
    // ---- operand splitters, then the first half of the epilogue
    const int t = threadIdx.x - 64;                             // 0 .. PO_WORKERS-1
    // The epilogue's per-row tables (permutation entries, bias noise, bias) are cold in HBM.  The first PO_PRE
    // chunks of this thread are loaded into registers now, where the whole K loop hides the latency; what lies
    // beyond is at least started on its way to L2.
    if (gm < p.B) {
      const long long d = gm % p.D;
#pragma unroll
      for (int ci = 0; ci < PO_PRE; ++ci) {
        const int c = chunk0 * 16 + ci * 32;
        const int k0 = kbase + c;
        if (c < p.NB && k0 + 16 <= p.out) {
          if (p.pout && p.vec_pout) {
            const uint4* pr = reinterpret_cast<const uint4*>(p.pout + d * p.out + k0);
            pre_so[ci][0] = __ldg(pr); pre_so[ci][1] = __ldg(pr + 1);
          }
          if (p.beta && p.vec_beta) {
            const float4* br = reinterpret_cast<const float4*>(p.beta + d * p.out + k0);
#pragma unroll
            for (int u = 0; u < 4; ++u) pre_bn[ci][u] = __ldg(br + u);
          }
          if (p.bias && p.vec_bias) {
            const float4* br = reinterpret_cast<const float4*>(p.bias + k0);
#pragma unroll
            for (int u = 0; u < 4; ++u) pre_bias[ci][u] = __ldg(br + u);
          }
        }
      }
      for (int c = chunk0 * 16 + PO_PRE * 32; c < p.NB && kbase + c < p.out; c += 32) {
        if (p.pout) prefetch_l2(p.pout + d * p.out + kbase + c);
        if (p.beta) prefetch_l2(p.beta + d * p.out + kbase + c);
      }
    }
    bool ok = true;
    for (int kt = 0; kt < nk && ok; ++kt) {
      const int s = kt % p.stages;
      const uint32_t ph = (kt / p.stages) & 1;
      ok = mbar_wait_relaxed(&full[s], ph, 4);
      if (!ok) break;
      PO_TRACE(kt == 0 && t == 0, 3);
      unsigned char* st = tiles + size_t(s) * stage_bytes;
      float4* a_hi = reinterpret_cast<float4*>(st);
      float4* a_lo = reinterpret_cast<float4*>(st + PO_A_BYTES);
      float4* b_hi = reinterpret_cast<float4*>(st + (TERMS == 3 ? 2 : 1) * PO_A_BYTES);
      float4* b_lo = reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(b_hi) + b_bytes);
#pragma unroll
      for (int u = 0; u < PO_A_BYTES / 16 / PO_WORKERS; ++u) {
        const int i = t + u * PO_WORKERS;
        const float4 v = a_hi[i];
        const float4 h = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
        a_hi[i] = h;
        if (TERMS == 3) a_lo[i] = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
      }
      for (int i = t; i < b_bytes / 16; i += PO_WORKERS) {
        const float4 v = b_hi[i];
        const float4 h = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
        b_hi[i] = h;
        if (TERMS == 3) b_lo[i] = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
      }
      fence_proxy_async_smem();                                 // these writes are read by tcgen05.mma (async proxy)
      __syncwarp();
      if (lane == 0) mbar_arrive(&split[s]);
      PO_TRACE(kt == 0 && t == 0, 4);
    }
    // noise accumulator -> this block's slice of the exchange area (the stage ring is free once every MMA has completed)
    const bool done = mbar_wait_relaxed(accum, 0, 3);
    PO_TRACE(t == 0, 7);
    tc_fence_after();
    if (done && nk > 0) {
      float* prow = my_slice + size_t(row) * pitch;
      for (int c = chunk0 * 16; c < p.NP; c += 32) {
        uint32_t r[16];
        tmem_ld16_nowait(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(p.NB + c), r);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 16; u += 4)
          *reinterpret_cast<float4*>(prow + c + u) = make_float4(__uint_as_float(r[u]), __uint_as_float(r[u + 1]),
                                                                 __uint_as_float(r[u + 2]), __uint_as_float(r[u + 3]));
      }
      if (p.local_gather) fence_proxy_async_smem();             // the slice is about to be read by bulk copies
    }
    PO_TRACE(t == 0, 8);
  }
  static_assert(PO_A_BYTES / 16 % PO_WORKERS == 0, "the A tile must split evenly over the splitter threads");
  __syncthreads();                       // re-converges the single-thread roles before the warp-aligned cluster barrier
  cluster_sync_all();                    // every block has finished its MMAs and written its slice
  PO_TRACE(threadIdx.x == 64, 9);

  if (p.local_gather && S > 1 && threadIdx.x == 64) {
    // push this block's slice into the same place of every peer; each block's xbar counts what it receives
    const uint32_t bytes = slice_floats * 4u;
    mbar_expect_tx(xbar, uint32_t(S - 1) * bytes);
    const uint32_t src = smem_u32(my_slice), bar = smem_u32(xbar);
    for (int r = 1; r < S; ++r) {
      const uint32_t peer = (j + uint32_t(r)) % uint32_t(S);
      bulk_push(map_to_rank(src, peer), src, bytes, map_to_rank(bar, peer));
    }
  }

  if (warp >= 2) {
    bool arrived = true;
    if (p.local_gather && S > 1) arrived = mbar_wait_relaxed(xbar, 0, 3);
    PO_TRACE(threadIdx.x == 64, 12);
    const bool live = arrived && (timeouts_so_far() == timeouts_at_start) && nk > 0;
    const bool row_ok = live && gm < p.B;
    long long d = 0;
    float sgn = 1.f;
    if (row_ok) { d = gm % p.D; sgn = anti_sign(gm / p.D, p.R, p.antithetic); }
    const float* lrow = xchg + size_t(row) * pitch;                       // local gather: + owner * slice_floats + column
    const uint32_t xrow = smem_u32(xchg) + uint32_t(row) * uint32_t(pitch) * 4u;
#pragma unroll 2
    for (int c = chunk0 * 16; c < p.NB; c += 32) {
      const int k0 = kbase + c;
      if (k0 >= p.out) break;                                    // uniform over the warp
      const int ci = (c - chunk0 * 16) >> 5;
      uint32_t acc[16];
      tmem_ld16_nowait(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(c), acc);
      tmem_ld_wait();
      if (!row_ok) continue;
      const bool whole = (k0 + 16 <= p.out);
      int so[16];
      if (p.pout) {
        const int16_t* pr = p.pout + d * p.out + k0;
        if (whole && p.vec_pout) {
          uint4 v0, v1;
          if (ci == 0) { v0 = pre_so[0][0]; v1 = pre_so[0][1]; }
          else if (ci == 1) { v0 = pre_so[1][0]; v1 = pre_so[1][1]; }
          else { v0 = __ldg(reinterpret_cast<const uint4*>(pr)); v1 = __ldg(reinterpret_cast<const uint4*>(pr) + 1); }
          const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
          for (int u = 0; u < 8; ++u) { so[2 * u] = int(w[u] & 0xFFFFu); so[2 * u + 1] = int(w[u] >> 16); }
        } else {
#pragma unroll
          for (int u = 0; u < 16; ++u) so[u] = (k0 + u < p.out) ? int(uint16_t(pr[u])) : 0x7FFF;
        }
      } else {
#pragma unroll
        for (int u = 0; u < 16; ++u) so[u] = k0 + u;
      }
      float qv[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        qv[u] = 0.f;
        if (so[u] < p.out_sp) {
          const uint32_t owner = __umulhi(uint32_t(so[u]), p.np_magic);
          const uint32_t col = uint32_t(so[u]) - owner * uint32_t(p.NP);
          if (p.local_gather) qv[u] = lrow[size_t(owner) * slice_floats + col];
          else qv[u] = ld_cluster_f32(xrow + col * 4u, owner);
        }
      }
      float bn[16];
      if (p.beta) {
        const float* br = p.beta + d * p.out + k0;
        if (whole && p.vec_beta) {
#pragma unroll
          for (int u = 0; u < 16; u += 4) {
            float4 v;
            if (ci == 0) v = pre_bn[0][u >> 2];
            else if (ci == 1) v = pre_bn[1][u >> 2];
            else v = __ldg(reinterpret_cast<const float4*>(br + u));
            bn[u] = v.x; bn[u + 1] = v.y; bn[u + 2] = v.z; bn[u + 3] = v.w;
          }
        } else {
#pragma unroll
          for (int u = 0; u < 16; ++u) bn[u] = (k0 + u < p.out) ? __ldg(br + u) : 0.f;
        }
      } else {
#pragma unroll
        for (int u = 0; u < 16; ++u) bn[u] = 0.f;
      }
      float bs[16];
      if (p.bias && whole && p.vec_bias && ci < PO_PRE) {
#pragma unroll
        for (int u = 0; u < 16; u += 4) {
          const float4 v = (ci == 0) ? pre_bias[0][u >> 2] : pre_bias[1][u >> 2];
          bs[u] = v.x; bs[u + 1] = v.y; bs[u + 2] = v.z; bs[u + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int u = 0; u < 16; ++u) bs[u] = (p.bias && k0 + u < p.out) ? __ldg(p.bias + k0 + u) : 0.f;
      }
      float o[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) o[u] = __uint_as_float(acc[u]) + bs[u] + sgn * (qv[u] + bn[u]);
      float* dst = p.y + gm * p.out + k0;
      if (whole && p.vec_y) {
#pragma unroll
        for (int u = 0; u < 16; u += 4) *reinterpret_cast<float4*>(dst + u) = make_float4(o[u], o[u + 1], o[u + 2], o[u + 3]);
      } else {
#pragma unroll
        for (int u = 0; u < 16; ++u) if (k0 + u < p.out) dst[u] = o[u];
      }
    }
  }
  PO_TRACE(threadIdx.x == 64, 10);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                    // no block leaves while a peer may still read or fill its exchange area
  PO_TRACE(threadIdx.x == 64, 11);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, uint32_t(p.tmem_cols));
  }
}

#ifdef NES_PO_TRACE
int po_trace_read(long long* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_po_trace, sizeof(long long) * 64 * 16);
  return e == cudaSuccess ? NES_OK : fail(NES_ERR_LAUNCH, "po_trace: %s", cudaGetErrorString(e));
}
#endif

int permuted_out_error_word(int* v, bool clear) { return read_error_word(v, clear, "tc_error_flag"); }

static int encode_rows(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int box_rows, const char* what) {
  EncodeTiledFn fn = encode_fn();
  NES_REQUIRE(fn != nullptr, NES_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", what);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
  cuuint32_t box[2] = {(cuuint32_t)PO_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NES_REQUIRE(r == CUDA_SUCCESS, NES_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
  return NES_OK;
}

static int ceil16(int64_t v) { return int((v + 15) & ~int64_t(15)); }

struct PermOutPlan { int S, NB, NP, stages, tmem_cols, local_gather; size_t smem; };

// Column split: S blocks per 128-row tile.  A block's MMAs take about max(92, 0.74 * N) cycles each
// (measured: an M128 kind::tf32 MMA is issue-bound below N = 128), so the split that minimises
// waves * that time is taken, the smaller S on a near-tie.
static bool plan_perm_out(int64_t B, int64_t out, int64_t out_sp, int64_t K, int terms, PermOutPlan* best) {
  const int64_t mtiles = ceil_div<int64_t>(B, PO_BM);
  const int sms = sm_count();
  double best_cost = 0.0;
  bool found = false;
  for (int S = 1; S <= 8; S *= 2) {
    PermOutPlan c;
    c.S = S;
    c.NB = ceil16(ceil_div<int64_t>(out, S));
    c.NP = ceil16(ceil_div<int64_t>(out_sp, S));
    const int NC = c.NB + c.NP;
    if (NC > 256) continue;
    const double per_mma = NC * 0.74 > 92.0 ? NC * 0.74 : 92.0;
    const double cost = double(ceil_div<int64_t>(mtiles * S, sms)) * per_mma;
    if (found && cost > best_cost * 0.95) continue;
    const int nk = int(ceil_div<int64_t>(K, PO_BK));
    const int stage_bytes = (terms == 3 ? 2 : 1) * (PO_A_BYTES + NC * PO_BK * 4);
    const size_t budget = 227 * 1024 - 1024 - 256;
    int stages = int(budget / stage_bytes);
    if (stages > 4) stages = 4;
    if (stages > nk) stages = nk;
    if (stages < 1) stages = 1;
    const size_t slice = size_t(PO_BM) * (c.NP + 4) * 4;
    c.local_gather = (slice * S <= budget) ? 1 : 0;            // the whole 128 x out_sp noise tile fits: gather locally
    const size_t xchg = c.local_gather ? slice * S : slice;
    size_t body = size_t(stages) * stage_bytes;
    if (xchg > body) body = xchg;
    if (body > budget) continue;
    c.stages = stages;
    c.smem = 1024 + ((body + 15) & ~size_t(15)) + (3 * stages + 2) * sizeof(uint64_t) + 16;
    if (c.smem < size_t(PO_MIN_SMEM)) c.smem = PO_MIN_SMEM;
    c.tmem_cols = 32;
    while (c.tmem_cols < NC) c.tmem_cols <<= 1;
    *best = c;
    best_cost = cost;
    found = true;
  }
  return found;
}

template <int TERMS>
static int launch_perm_out(const PermOutParams& prm, const PermOutPlan& plan, int64_t mtiles, cudaStream_t st) {
  auto kern = permuted_linear_out_kernel<TERMS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "permuted_linear_out_fwd_tc: shared memory opt-in failed: %s", cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)plan.S, (unsigned)mtiles, 1);
  cfg.blockDim = dim3(PO_THREADS, 1, 1);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)plan.S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, prm);
  count_launch();
  if (e != cudaSuccess) return fail(NES_ERR_LAUNCH, "permuted_linear_out_fwd_tc: %s", cudaGetErrorString(e));
  return NES_OK;
}

}  // namespace tc
}  // namespace nes

using namespace nes;
using namespace nes::tc;

extern "C" int nes_permuted_linear_out_fwd_tc_supported(int64_t D, int64_t R, int64_t in, int64_t out, int64_t out_sp, int mode) {
  if (D <= 0 || R <= 0 || in <= 0 || out <= 0 || out_sp <= 0 || out_sp > out) return 0;
  if (mode != 1 && mode != 3) return 0;
  if (in % 4 != 0 || in > INT32_MAX - 64 || out > 32767 || D * R > INT32_MAX - 256) return 0;
  if (ceil_div<int64_t>(D * R, PO_BM) > 65535) return 0;
  PermOutPlan plan;
  return plan_perm_out(D * R, out, out_sp, in, mode, &plan) ? 1 : 0;
}

extern "C" int nes_permuted_linear_out_fwd_tc(const float* x, const float* weight, const float* bias, const float* eps,
                                              const float* bias_noise, const int16_t* pout, float* y,
                                              int64_t D, int64_t R, int64_t in, int64_t out, int64_t out_sp,
                                              int antithetic, int mode, nes_stream_t stream) {
  NES_REQUIRE(D >= 0 && R >= 0 && in >= 0 && out >= 0 && out_sp >= 0 && out_sp <= out, NES_ERR_BAD_ARG,
              "permuted_linear_out_fwd_tc: bad extent");
  NES_REQUIRE(mode == 1 || mode == 3, NES_ERR_BAD_ARG, "permuted_linear_out_fwd_tc: mode must be 1 (TF32) or 3 (3xTF32)");
  if (D == 0 || R == 0 || out == 0) return NES_OK;
  NES_REQUIRE(x && weight && eps && y, NES_ERR_BAD_ARG, "permuted_linear_out_fwd_tc: null pointer");
  NES_REQUIRE(pout || out_sp == out, NES_ERR_BAD_ARG, "permuted_linear_out_fwd_tc: out_sp != out without output permutations");
  NES_REQUIRE(nes_permuted_linear_out_fwd_tc_supported(D, R, in, out, out_sp, mode), NES_ERR_UNSUPPORTED,
              "permuted_linear_out_fwd_tc: shape D=%lld R=%lld in=%lld out=%lld out_sp=%lld is not covered (in must be a positive "
              "multiple of 4, out + out_sp <= 2048)", (long long)D, (long long)R, (long long)in, (long long)out, (long long)out_sp);
  NES_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(eps), NES_ERR_UNSUPPORTED,
              "permuted_linear_out_fwd_tc: x, weight and eps must be 16-byte aligned (TMA)");
  const int64_t B = D * R;
  PermOutPlan plan;
  plan_perm_out(B, out, out_sp, in, mode, &plan);
  PermOutParams prm;
  int rc;
  if ((rc = encode_rows(&prm.map_x, x, B, in, PO_BM, "permuted_linear_out_fwd_tc")) != NES_OK) return rc;
  if ((rc = encode_rows(&prm.map_w, weight, out, in, plan.NB, "permuted_linear_out_fwd_tc")) != NES_OK) return rc;
  if ((rc = encode_rows(&prm.map_eps, eps, out_sp, in, plan.NP, "permuted_linear_out_fwd_tc")) != NES_OK) return rc;
  prm.bias = bias; prm.beta = bias_noise; prm.pout = pout; prm.y = y;
  prm.B = B; prm.D = D; prm.R = R;
  prm.out = int(out); prm.out_sp = int(out_sp); prm.K = int(in);
  prm.NB = plan.NB; prm.NP = plan.NP;
  prm.stages = plan.stages; prm.tmem_cols = plan.tmem_cols; prm.antithetic = antithetic;
  prm.np_magic = (unsigned int)((0x100000000ULL + uint64_t(plan.NP) - 1) / uint64_t(plan.NP));
  prm.vec_y = (out % 4 == 0) && aligned16(y);
  prm.vec_pout = pout && (out % 8 == 0) && aligned16(pout);
  prm.vec_beta = bias_noise && (out % 4 == 0) && aligned16(bias_noise);
  prm.vec_bias = bias && aligned16(bias);
  prm.local_gather = plan.local_gather;
  const int64_t mtiles = ceil_div<int64_t>(B, PO_BM);
  cudaStream_t st = as_stream(stream);
  return mode == 3 ? launch_perm_out<3>(prm, plan, mtiles, st) : launch_perm_out<1>(prm, plan, mtiles, st);
}

#ifdef NES_PO_TRACE
// instrumented builds only: copies the 64 x 16 phase timestamps of the last launches to host memory
extern "C" int nes_debug_po_trace(long long* out) { return nes::tc::po_trace_read(out); }
#endif
