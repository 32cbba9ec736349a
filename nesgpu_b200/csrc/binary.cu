// Bit-packed ("binary") kernels: packing, Bernoulli bit sampling, XOR-popcount batched
// matrix products (plain, thresholded, and convolution without materialised columns),
// fitness-weighted bit sums and OR max-pooling.  Integer work on CUDA cores (LOP3 + POPC),
// bounded by HBM for everything except the weighted sum, which is bounded by the per-bit
// predicated adds.
#include "common.cuh"

namespace nes {

__device__ inline int popc_word(uint32_t v) { return __popc(v); }
__device__ inline int popc_word(uint64_t v) { return __popcll(v); }

// eight bool bytes (any non-zero value counts as true) -> eight bits, byte i -> bit i
__device__ inline uint32_t squeeze8(uint64_t x) {
  x = ((((x & 0x7F7F7F7F7F7F7F7FULL) + 0x7F7F7F7F7F7F7F7FULL) | x) >> 7) & 0x0101010101010101ULL;
  return uint32_t((x * 0x0002040810204081ULL) >> 49) & 0xFFu;
}
// eight bits -> eight bool bytes (0/1)
__device__ inline uint64_t spread8(uint32_t b) {
  uint64_t y = (uint64_t(b & 0xFFu) * 0x0101010101010101ULL) & 0x8040201008040201ULL;
  return ((y + 0x7F7F7F7F7F7F7F7FULL) >> 7) & 0x0101010101010101ULL;
}

// ---- pack / unpack ----------------------------------------------------------------------
// One thread produces one output byte = eight input columns; out_row_bytes is the padded
// row length (words * word_bytes), bytes past ceil(cols/8) are zero.
template <bool BYTES>   // BYTES: int8pack (copy bytes) instead of squeezing bools
__global__ void pack_rows_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t rows,
                                 int64_t cols, int64_t out_row_bytes, int aligned8) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= rows * out_row_bytes) return;
  const int64_t r = e / out_row_bytes, g = e - r * out_row_bytes;
  if (BYTES) {
    out[e] = (g < cols) ? in[r * cols + g] : uint8_t(0);
    return;
  }
  const int64_t c0 = g * 8;
  uint64_t x = 0;
  if (c0 + 8 <= cols && aligned8) {
    x = *reinterpret_cast<const uint64_t*>(in + r * cols + c0);
  } else {
    for (int i = 0; i < 8; ++i)
      if (c0 + i < cols) x |= uint64_t(in[r * cols + c0 + i]) << (8 * i);
  }
  out[e] = uint8_t(squeeze8(x));
}

__global__ void unpack_rows_kernel(const uint8_t* __restrict__ in, uint64_t* __restrict__ out, int64_t nbytes) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= nbytes) return;
  out[e] = spread8(in[e]);
}

// ---- Bernoulli bit sampling -------------------------------------------------------------
// Injected uniforms: one thread produces 32 output bits of member x, row y (bit = p > u).
__global__ void sample_bits_kernel(const __half* __restrict__ p, const float* __restrict__ u,
                                   uint32_t* __restrict__ out, int64_t n, int64_t rows, int64_t cols,
                                   int64_t row_u32, uint64_t seed, int vec) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= n * rows * row_u32) return;
  const int64_t q = e % row_u32;
  const int64_t xy = e / row_u32;
  const int64_t y = xy % rows, x = xy / rows;
  const int64_t c0 = q * 32;
  uint32_t word = 0;
  if (c0 < cols) {
    const __half* pr = p + y * cols + c0;
    const int lim = int(cols - c0 < 32 ? cols - c0 : 32);
    const float* ur = u + xy * cols + c0;
    if (vec && lim == 32) {
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float4 uv = __ldcs(reinterpret_cast<const float4*>(ur) + g);
        const uint2 pv = __ldg(reinterpret_cast<const uint2*>(pr) + g);
        const __half2 p01 = *reinterpret_cast<const __half2*>(&pv.x);
        const __half2 p23 = *reinterpret_cast<const __half2*>(&pv.y);
        word |= uint32_t(__low2float(p01) > uv.x) << (4 * g);
        word |= uint32_t(__high2float(p01) > uv.y) << (4 * g + 1);
        word |= uint32_t(__low2float(p23) > uv.z) << (4 * g + 2);
        word |= uint32_t(__high2float(p23) > uv.w) << (4 * g + 3);
      }
    } else {
      for (int i = 0; i < lim; ++i) word |= uint32_t(__half2float(pr[i]) > ur[i]) << i;
    }
  }
  out[e] = word;
}

// Device-generated variant: one thread owns 32 columns of one row and walks a chunk of members.  A bit
// is set when a 16-bit uniform integer U is below T = ceil(p * 65536), i.e. with probability p rounded
// up to a multiple of 2^-16 (p = 0 never, p = 1 always).  The comparison runs on all 32 columns at once,
// bit-sliced: the thresholds are held as 16 bit-planes (plane j, bit i = bit j of T_i), a random word
// supplies bit j of all 32 uniforms, and from the top plane down a column is decided at the first plane
// where its uniform and its threshold differ.  Two Philox-4x32 calls of seven rounds per word (the kernel is bound by
// this integer arithmetic; seven is the smallest count the generator's authors report as passing BigCrush; counter = (column
// group, row, member)) give eight words: word k is bit 15-k of the uniforms, and the same word rotated
// by k+1 columns is bit 7-k, so each U is sixteen independent random bits (its low byte is made of bits
// that serve as high-byte bits of other columns; it only matters when the high bytes of U and T agree).
struct BitDrawer {
  uint32_t plane[16];
  uint32_t always;

  __device__ inline void init(const __half* __restrict__ p, int64_t y, int64_t c0, int64_t cols) {
#pragma unroll
    for (int j = 0; j < 16; ++j) plane[j] = 0u;
    always = 0u;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float pv = 0.f;
      if (c0 + i < cols) pv = __half2float(p[y * cols + c0 + i]);
      const float t = ceilf(pv * 65536.f);
      const uint32_t T = (t <= 0.f) ? 0u : (t >= 65536.f ? 65536u : uint32_t(t));
      always |= (T >> 16) << i;
#pragma unroll
      for (int j = 0; j < 16; ++j) plane[j] |= ((T >> j) & 1u) << i;
    }
  }

  __device__ inline uint32_t draw(const Philox& ph, int64_t q, int64_t y, int64_t x) const {
    uint32_t r[8];
    ph.rounds<7>(uint32_t(q * 2), uint32_t(y), uint32_t(x), 5u, r);
    ph.rounds<7>(uint32_t(q * 2 + 1), uint32_t(y), uint32_t(x), 5u, r + 4);
    uint32_t und = ~0u, res = always;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t P = plane[15 - k];
      const uint32_t diff = r[k] ^ P;
      res |= und & diff & P;
      und &= ~diff;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t P = plane[7 - k];
      const uint32_t diff = __funnelshift_r(r[k], r[k], k + 1) ^ P;
      res |= und & diff & P;
      und &= ~diff;
    }
    return res;
  }
};

__global__ void __launch_bounds__(256) sample_bits_philox_kernel(const __half* __restrict__ p, uint32_t* __restrict__ out,
                                                                 int64_t n, int64_t rows, int64_t cols, int64_t row_u32,
                                                                 uint64_t seed, int members) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= rows * row_u32) return;
  const int64_t q = e % row_u32, y = e / row_u32;
  BitDrawer bd;
  bd.init(p, y, q * 32, cols);
  const Philox ph(seed);
  const int64_t x0 = int64_t(blockIdx.y) * members;
  const int64_t x1 = (x0 + members < n) ? x0 + members : n;
  for (int64_t x = x0; x < x1; ++x) out[(x * rows + y) * row_u32 + q] = bd.draw(ph, q, y, x);
}

// Fused sampling + product: the weight bits of member x are drawn exactly as sample_bits_philox_kernel draws
// them (same counters, same thresholds) and consumed on the spot,
//   C[x, y] = sum_z popcount(bits(x, y, z) ^ B[x, z]),
// so the (n, rows, words) bit tensor is never stored.  Integer atomics make the sum order-independent.
__global__ void __launch_bounds__(256) seeded_bmv_kernel(const __half* __restrict__ p, const uint32_t* __restrict__ B,
                                                         int32_t* __restrict__ C, int64_t n, int64_t rows, int64_t cols,
                                                         int64_t row_u32, uint64_t seed, int members) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= rows * row_u32) return;
  const int64_t q = e % row_u32, y = e / row_u32;
  BitDrawer bd;
  bd.init(p, y, q * 32, cols);
  const Philox ph(seed);
  const int64_t x0 = int64_t(blockIdx.y) * members;
  const int64_t x1 = (x0 + members < n) ? x0 + members : n;
  for (int64_t x = x0; x < x1; ++x) {
    const uint32_t word = bd.draw(ph, q, y, x);
    int cnt = __popc(word ^ __ldg(B + x * row_u32 + q));
    // lanes of a warp hold consecutive 32-bit columns; when a row is a whole number of warps wide the
    // warp reduces first and issues one atomic
    if ((row_u32 & 31) == 0) {
#pragma unroll
      for (int sh = 16; sh > 0; sh >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, sh);
      if ((threadIdx.x & 31) == 0) atomicAdd(C + x * rows + y, cnt);
    } else {
      atomicAdd(C + x * rows + y, cnt);
    }
  }
}

// Members per block for the two kernels above: the threshold planes cost about a thousand instructions
// to set up, so a block keeps them for as many members as still leaves the grid a few waves deep.
static int sample_members_per_block(int64_t n, int64_t column_blocks) {
  int m = 64;
  while (m > 8 && column_blocks * ceil_div<int64_t>(n, m) < int64_t(sm_count()) * 8) m >>= 1;
  return m;
}

// ---- XOR-popcount batched matrix product ------------------------------------------------

struct DirectA {   // A (P, M, K) words
  const void* A; int64_t M; int K;
  template <typename T>
  __device__ inline T load(int64_t z, int64_t m, int k) const {
    return (m < M && k < K) ? static_cast<const T*>(A)[(z * M + m) * K + k] : T(0);
  }
};

struct WindowA {   // implicit im2col of packed NHWC (P,H,W,Cw): m = (xo,yo), k = ((i*fy)+j)*Cw + c
  const void* in; int H, W, Cw, fx, fy, px, py, sx, sy, wo; int64_t M; int K;
  template <typename T>
  __device__ inline T load(int64_t z, int64_t m, int k) const {
    if (m >= M || k >= K) return T(0);
    const int tap = k / Cw, c = k - tap * Cw;
    const int i = tap / fy, j = tap - i * fy;
    const int xo = int(m / wo), yo = int(m - int64_t(xo) * wo);
    const int xi = i + xo * sx - px, yi = j + yo * sy - py;
    if (xi < 0 || xi >= H || yi < 0 || yi >= W) return T(0);
    return static_cast<const T*>(in)[((z * H + xi) * W + yi) * Cw + c];
  }
};

struct CountEpi {
  int32_t* C;
  __device__ inline void operator()(int64_t z, int64_t idx, int, int64_t, int acc) const { C[idx] = acc; }
};
struct ThreshEpi {   // 2*acc > thresh[z, n]
  uint8_t* C; const int32_t* thresh;
  __device__ inline void operator()(int64_t z, int64_t idx, int n, int64_t N, int acc) const {
    C[idx] = uint8_t(2 * acc > thresh[z * N + n]);
  }
};

constexpr int BT = 64, BKW = 8;   // 64x64 output tile, 8 words of K per step

template <typename T, class ALoad, class Epi>
__global__ void __launch_bounds__(256) bin_gemm_kernel(const ALoad al, const T* __restrict__ B, const Epi epi,
                                                       int64_t M, int K, int64_t N) {
  __shared__ T As[BKW][BT + 2];
  __shared__ T Bs[BKW][BT];
  const int t = threadIdx.x;
  const int64_t z = blockIdx.z;
  const int64_t m0 = int64_t(blockIdx.y) * BT, n0 = int64_t(blockIdx.x) * BT;
  const int tm = t >> 4, tn = t & 15;
  int acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0;
  for (int k0 = 0; k0 < K; k0 += BKW) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = (t >> 3) + 32 * i, k = t & 7;
      As[k][r] = al.template load<T>(z, m0 + r, k0 + k);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = (t >> 6) + 4 * i, n = t & 63;
      Bs[k][n] = (k0 + k < K && n0 + n < N) ? B[(z * K + k0 + k) * N + n0 + n] : T(0);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BKW; ++k) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][tm * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tn * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += popc_word(T(a[i] ^ b[j]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + tm * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tn * 4 + j;
      if (n < N) epi(z, (z * M + m) * N + n, int(n), N, acc[i][j]);
    }
  }
}

// N == 1 (one bit vector per member against that member's weight rows): pure streaming of A.
// Rows are cut into 16-byte chunks; a thread XORs a chunk with the matching chunk of the
// member's vector (shared memory), popcounts, and the chunks of a row are combined with
// segmented shuffles (chunks-per-row is a power of two <= 32 here).
template <class Epi>
__global__ void __launch_bounds__(256) bin_bmv_kernel(const uint4* __restrict__ A, const uint4* __restrict__ B,
                                                      const Epi epi, int64_t M, int cpr /*chunks per row*/,
                                                      int rows_per_block) {
  extern __shared__ __align__(16) unsigned char dyn[];
  uint4* bs = reinterpret_cast<uint4*>(dyn);
  const int64_t z = blockIdx.y;
  const int64_t r0 = int64_t(blockIdx.x) * rows_per_block;
  for (int c = threadIdx.x; c < cpr; c += blockDim.x) bs[c] = B[z * cpr + c];
  __syncthreads();
  const int64_t rows_here = (M - r0 < rows_per_block) ? (M - r0) : rows_per_block;
  const int64_t chunks = rows_here * cpr;
  const uint4* a = A + (z * M + r0) * cpr;
  const int64_t iters = ceil_div<int64_t>(chunks, 256);
  for (int64_t it = 0; it < iters; it += 4) {
    uint4 v[4];
    int64_t g[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      g[u] = (it + u) * 256 + threadIdx.x;
      v[u] = (it + u < iters && g[u] < chunks) ? __ldcs(a + g[u]) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (it + u >= iters) break;                  // uniform across the block
      const bool ok = g[u] < chunks;
      const int c = ok ? int(g[u] % cpr) : 0;
      const uint4 b = bs[c];
      int s = ok ? (__popc(v[u].x ^ b.x) + __popc(v[u].y ^ b.y) + __popc(v[u].z ^ b.z) + __popc(v[u].w ^ b.w)) : 0;
      for (int sh = cpr >> 1; sh > 0; sh >>= 1) s += __shfl_down_sync(0xffffffffu, s, sh, cpr);
      if (ok && c == 0) {
        const int64_t m = r0 + g[u] / cpr;
        epi(z, z * M + m, 0, 1, s);
      }
    }
  }
}

// ---- materialised im2col (API parity) and OR max-pool --------------------------------------
template <typename T>
__global__ void im2col_kernel(const WindowA wa, T* __restrict__ out, int64_t total) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int k = int(e % wa.K);
  const int64_t zm = e / wa.K;
  out[e] = wa.template load<T>(zm / wa.M, zm % wa.M, k);
}

template <typename T>
__global__ void maxpool_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t total, int H, int W,
                               int Cw, int ho, int wo, int px, int py, int sx, int sy) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int c = int(e % Cw);
  int64_t r = e / Cw;
  const int yo = int(r % wo); r /= wo;
  const int xo = int(r % ho);
  const int64_t z = r / ho;
  T v = 0;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int xi = i + xo * sx - px, yi = j + yo * sy - py;
      if (xi >= 0 && xi < H && yi >= 0 && yi < W) v |= in[((z * H + xi) * W + yi) * Cw + c];
    }
  out[e] = v;
}

// ---- fitness-weighted bit sum ------------------------------------------------------------
// Data is viewed as 32-bit columns (little-endian, so bit z of a row is bit z%32 of column
// z/32 for both word widths).  A block owns one output row and up to 256 columns; its threads
// are (member slot, column) pairs, each keeping 32 fp32 accumulators and walking its members
// with four loads in flight.  Slots are combined through shared memory 16 bits at a time;
// blockIdx.z splits the members, with fp32 partial rows in scratch summed by a last kernel.
//
// When every warp holds one member slot (column count per block a multiple of 32) members are
// taken four at a time: the four words are bit-transposed so that each nibble holds the four
// members' bits of one position, and the nibble selects one of the 16 subset sums of the four
// weights, which the lanes of the warp hold (lane & 15) and hand out by shuffle.  One shift,
// one shuffle and one add then cover four member-bits.  (A 16-entry shared-memory table in
// place of the shuffle measured slower: 102 us against 81 us at 1024 members of 1024x1024 bits.)
constexpr int WS_THREADS = 256;

template <bool QUAD>
__global__ void __launch_bounds__(WS_THREADS) weighted_sum_kernel(
    const uint32_t* __restrict__ in, const __half* __restrict__ w, float* __restrict__ partial,
    int64_t D, int64_t rows, int row_u32, int64_t zbits, int64_t d_per_split, int cols_per_block, int slots) {
  __shared__ float red[WS_THREADS][17];
  const int t = threadIdx.x;
  const int col_l = t % cols_per_block, slot = t / cols_per_block;
  const int col = blockIdx.x * cols_per_block + col_l;
  const int64_t y = blockIdx.y;
  const int64_t d0 = blockIdx.z * d_per_split;
  const int64_t d1 = (d0 + d_per_split < D) ? d0 + d_per_split : D;
  const bool active = (slot < slots) && (col < row_u32);
  float acc[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) acc[i] = 0.f;
  if (active) {
    const uint32_t* src = in + y * row_u32 + col;
    const int64_t stride = rows * row_u32;
    int64_t d = d0 + slot;
    if (QUAD) {
      const int e = t & 15;
      const int64_t quads = (d1 - d0) / 4;
      uint32_t n0 = 0, n1 = 0, n2 = 0, n3 = 0;
      if (slot < quads) {
        const int64_t db = d0 + 4 * int64_t(slot);
        n0 = __ldcs(src + db * stride); n1 = __ldcs(src + (db + 1) * stride);
        n2 = __ldcs(src + (db + 2) * stride); n3 = __ldcs(src + (db + 3) * stride);
      }
      for (int64_t g = slot; g < quads; g += slots) {
        const int64_t db = d0 + 4 * g;
        const uint32_t a0 = n0, a1 = n1, a2 = n2, a3 = n3;
        if (g + slots < quads) {            // next group's words fly while this one is summed
          const int64_t dn = db + 4 * int64_t(slots);
          n0 = __ldcs(src + dn * stride); n1 = __ldcs(src + (dn + 1) * stride);
          n2 = __ldcs(src + (dn + 2) * stride); n3 = __ldcs(src + (dn + 3) * stride);
        }
        float lut = (e & 1) ? __half2float(w[db]) : 0.f;
        lut += (e & 2) ? __half2float(w[db + 1]) : 0.f;
        lut += (e & 4) ? __half2float(w[db + 2]) : 0.f;
        lut += (e & 8) ? __half2float(w[db + 3]) : 0.f;
        // 4x4 bit transposes: nibble k of u[tt] = members' bits (m3 m2 m1 m0) of position 4k + tt
        const uint32_t b0 = (a0 & 0x55555555u) | ((a1 & 0x55555555u) << 1);
        const uint32_t b1 = ((a0 >> 1) & 0x55555555u) | (a1 & 0xAAAAAAAAu);
        const uint32_t b2 = (a2 & 0x55555555u) | ((a3 & 0x55555555u) << 1);
        const uint32_t b3 = ((a2 >> 1) & 0x55555555u) | (a3 & 0xAAAAAAAAu);
        uint32_t u[4];
        u[0] = (b0 & 0x33333333u) | ((b2 & 0x33333333u) << 2);
        u[2] = ((b0 >> 2) & 0x33333333u) | (b2 & 0xCCCCCCCCu);
        u[1] = (b1 & 0x33333333u) | ((b3 & 0x33333333u) << 2);
        u[3] = ((b1 >> 2) & 0x33333333u) | (b3 & 0xCCCCCCCCu);
#pragma unroll
        for (int k = 0; k < 8; ++k)
#pragma unroll
          for (int tt = 0; tt < 4; ++tt)
            acc[4 * k + tt] += __shfl_sync(0xffffffffu, lut, int(u[tt] >> (4 * k)), 16);
      }
      d = d0 + 4 * quads + slot;
    }
    for (; d + 3 * slots < d1; d += 4 * slots) {
      uint32_t v[4]; float wd[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) { v[u] = __ldcs(src + (d + u * slots) * stride); wd[u] = __half2float(w[d + u * slots]); }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] += ((v[u] >> i) & 1u) ? wd[u] : 0.f;
    }
    for (; d < d1; d += slots) {
      const uint32_t v = __ldcs(src + d * stride);
      const float wd = __half2float(w[d]);
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] += ((v >> i) & 1u) ? wd : 0.f;
    }
  }
  float* dst = partial + (blockIdx.z * rows + y) * zbits;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 16; ++i) red[t][i] = acc[half * 16 + i];
    __syncthreads();
    for (int e = t; e < cols_per_block * 16; e += WS_THREADS) {
      const int cl = e >> 4, i = e & 15;
      const int64_t c = int64_t(blockIdx.x) * cols_per_block + cl;
      const int64_t zb = c * 32 + half * 16 + i;
      if (c < row_u32 && zb < zbits) {
        float s = 0.f;
        for (int sl = 0; sl < slots; ++sl) s += red[sl * cols_per_block + cl][i];
        dst[zb] = s;
      }
    }
  }
}

__global__ void weighted_sum_finish_kernel(const float* __restrict__ partial, __half* __restrict__ out,
                                           int splits, int64_t n) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= n) return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += partial[k * n + e];
  out[e] = __float2half(s);
}

struct WsPlan { int cols_per_block, slots, bx, splits; int64_t d_per_split; };
static WsPlan plan_weighted_sum(int64_t D, int64_t rows, int64_t row_u32) {
  WsPlan p;
  p.cols_per_block = int(row_u32 < WS_THREADS ? row_u32 : WS_THREADS);
  if (p.cols_per_block < 1) p.cols_per_block = 1;
  p.slots = WS_THREADS / p.cols_per_block;
  p.bx = int(ceil_div<int64_t>(row_u32, p.cols_per_block));
  const int64_t blocks = int64_t(p.bx) * rows;
  const int64_t want = int64_t(sm_count()) * 8;
  int64_t s = ceil_div<int64_t>(want, blocks > 0 ? blocks : 1);
  const int64_t cap = D / (int64_t(p.slots) * 8);    // keep >= 8 members per thread
  if (s > cap) s = cap;
  if (s > 16) s = 16;
  if (s < 1) s = 1;
  p.d_per_split = ceil_div<int64_t>(D, s);
  p.splits = int(ceil_div<int64_t>(D, p.d_per_split > 0 ? p.d_per_split : 1));
  if (p.splits < 1) p.splits = 1;
  return p;
}

template <typename T, class ALoad>
static int launch_bin_gemm(const ALoad& al, const void* B, const int32_t* thresh, int32_t* counts, uint8_t* bools,
                           int64_t P, int64_t M, int64_t K, int64_t N, cudaStream_t st, const char* what) {
  NES_REQUIRE(P <= 65535 && ceil_div<int64_t>(M, BT) <= 65535 && ceil_div<int64_t>(N, BT) <= INT32_MAX && K <= INT32_MAX,
              NES_ERR_UNSUPPORTED, "%s: extent too large", what);
  dim3 grid((unsigned)ceil_div<int64_t>(N, BT), (unsigned)ceil_div<int64_t>(M, BT), (unsigned)P);
  if (thresh) {
    ThreshEpi e; e.C = bools; e.thresh = thresh;
    bin_gemm_kernel<T, ALoad, ThreshEpi><<<grid, 256, 0, st>>>(al, static_cast<const T*>(B), e, M, int(K), N);
  } else {
    CountEpi e; e.C = counts;
    bin_gemm_kernel<T, ALoad, CountEpi><<<grid, 256, 0, st>>>(al, static_cast<const T*>(B), e, M, int(K), N);
  }
  return check_launch(what);
}

// row-streaming N = 1 product of the layer file (binary_layers.cu)
bool bmv_rows_covers(const void* A, const void* X, int64_t P, int64_t K, int word_bits);
int bmv_rows_counts(const void* A, const void* X, int32_t* counts, int64_t P, int64_t M, int64_t K, int word_bits, cudaStream_t st);

static int bin_bmm_common(const void* A, const void* B, const int32_t* thresh, int32_t* counts, uint8_t* bools,
                          int64_t P, int64_t M, int64_t K, int64_t N, int word_bits, cudaStream_t st,
                          const char* what) {
  NES_REQUIRE(P >= 0 && M >= 0 && K >= 0 && N >= 0, NES_ERR_BAD_ARG, "%s: negative extent", what);
  NES_REQUIRE(word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "%s: word_bits must be 32 or 64", what);
  if (P == 0 || M == 0 || N == 0) return NES_OK;
  NES_REQUIRE(A && B && (counts || bools), NES_ERR_BAD_ARG, "%s: null pointer", what);
  const int64_t row_bytes = K * (word_bits / 8);
  const int64_t cpr = row_bytes / 16;
  const bool pow2 = cpr > 0 && (cpr & (cpr - 1)) == 0;
  if (N == 1 && !thresh && bmv_rows_covers(A, B, P, K, word_bits)) return bmv_rows_counts(A, B, counts, P, M, K, word_bits, st);
  if (N == 1 && K > 0 && row_bytes % 16 == 0 && pow2 && cpr <= 32 && aligned16(A) && aligned16(B) && P <= 65535) {
    // streaming fast path
    const int rows_per_block = int(256 * 8 / cpr);   // eight 16-byte chunks per thread
    dim3 grid((unsigned)ceil_div<int64_t>(M, rows_per_block), (unsigned)P);
    const size_t smem = size_t(cpr) * sizeof(uint4);
    if (thresh) {
      ThreshEpi e; e.C = bools; e.thresh = thresh;
      bin_bmv_kernel<ThreshEpi><<<grid, 256, smem, st>>>(static_cast<const uint4*>(A), static_cast<const uint4*>(B), e, M, int(cpr), rows_per_block);
    } else {
      CountEpi e; e.C = counts;
      bin_bmv_kernel<CountEpi><<<grid, 256, smem, st>>>(static_cast<const uint4*>(A), static_cast<const uint4*>(B), e, M, int(cpr), rows_per_block);
    }
    return check_launch(what);
  }
  DirectA al; al.A = A; al.M = M; al.K = int(K);
  if (word_bits == 64) return launch_bin_gemm<uint64_t>(al, B, thresh, counts, bools, P, M, K, N, st, what);
  return launch_bin_gemm<uint32_t>(al, B, thresh, counts, bools, P, M, K, N, st, what);
}

static int make_window(WindowA& wa, const void* in, int64_t P, int H, int W, int Cw, int fx, int fy, int px, int py,
                       int sx, int sy, int& ho, int& wo, const char* what) {
  NES_REQUIRE(P >= 0 && H > 0 && W > 0 && Cw > 0 && fx > 0 && fy > 0 && px >= 0 && py >= 0 && sx > 0 && sy > 0,
              NES_ERR_BAD_ARG, "%s: bad geometry", what);
  ho = (H - fx + 2 * px) / sx + 1;
  wo = (W - fy + 2 * py) / sy + 1;
  NES_REQUIRE(ho > 0 && wo > 0, NES_ERR_BAD_ARG, "%s: empty output", what);
  wa.in = in; wa.H = H; wa.W = W; wa.Cw = Cw; wa.fx = fx; wa.fy = fy; wa.px = px; wa.py = py; wa.sx = sx; wa.sy = sy;
  wa.wo = wo; wa.M = int64_t(ho) * wo; wa.K = fx * fy * Cw;
  return NES_OK;
}

int bin_weighted_sum_impl(const void* in, const uint16_t* w_half, uint16_t* out_half, int64_t D, int64_t rows,
                          int64_t words, int64_t zbits, int word_bits, void* scratch, int64_t scratch_bytes,
                          cudaStream_t st);

}  // namespace nes

using namespace nes;

extern "C" int nes_bin_pack(const uint8_t* in, void* out, int64_t rows, int64_t cols, int word_bits,
                            nes_stream_t stream) {
  NES_REQUIRE(rows >= 0 && cols >= 0, NES_ERR_BAD_ARG, "bin_pack: negative extent");
  NES_REQUIRE(word_bits == 8 || word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "bin_pack: word_bits must be 8, 32 or 64");
  const int64_t row_bytes = ceil_div<int64_t>(cols, word_bits) * (word_bits / 8);
  const int64_t total = rows * row_bytes;
  if (total == 0) return NES_OK;
  NES_REQUIRE(in && out, NES_ERR_BAD_ARG, "bin_pack: null pointer");
  const int aligned8 = (cols % 8 == 0) && ((reinterpret_cast<uintptr_t>(in) & 7u) == 0);
  pack_rows_kernel<false><<<(unsigned)ceil_div<int64_t>(total, 256), 256, 0, as_stream(stream)>>>(
      in, static_cast<uint8_t*>(out), rows, cols, row_bytes, aligned8);
  return check_launch("bin_pack");
}

extern "C" int nes_bin_pack8(const uint8_t* in, int8_t* out, int64_t rows, int64_t cols, nes_stream_t stream) {
  return nes_bin_pack(in, out, rows, cols, 8, stream);
}

extern "C" int nes_bin_int8pack(const uint8_t* in, void* out, int64_t rows, int64_t cols, int word_bits,
                                nes_stream_t stream) {
  NES_REQUIRE(rows >= 0 && cols >= 0, NES_ERR_BAD_ARG, "bin_int8pack: negative extent");
  NES_REQUIRE(word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "bin_int8pack: word_bits must be 32 or 64");
  const int wb = word_bits / 8;
  const int64_t row_bytes = ceil_div<int64_t>(cols, wb) * wb;
  const int64_t total = rows * row_bytes;
  if (total == 0) return NES_OK;
  NES_REQUIRE(in && out, NES_ERR_BAD_ARG, "bin_int8pack: null pointer");
  pack_rows_kernel<true><<<(unsigned)ceil_div<int64_t>(total, 256), 256, 0, as_stream(stream)>>>(
      in, static_cast<uint8_t*>(out), rows, cols, row_bytes, 0);
  return check_launch("bin_int8pack");
}

extern "C" int nes_bin_unpack(const void* in, uint8_t* out, int64_t rows, int64_t words, int word_bits,
                              nes_stream_t stream) {
  NES_REQUIRE(rows >= 0 && words >= 0, NES_ERR_BAD_ARG, "bin_unpack: negative extent");
  NES_REQUIRE(word_bits == 8 || word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "bin_unpack: word_bits must be 8, 32 or 64");
  const int64_t nbytes = rows * words * (word_bits / 8);
  if (nbytes == 0) return NES_OK;
  NES_REQUIRE(in && out, NES_ERR_BAD_ARG, "bin_unpack: null pointer");
  NES_REQUIRE((reinterpret_cast<uintptr_t>(out) & 7u) == 0, NES_ERR_BAD_ARG, "bin_unpack: output must be 8-byte aligned");
  unpack_rows_kernel<<<(unsigned)ceil_div<int64_t>(nbytes, 256), 256, 0, as_stream(stream)>>>(
      static_cast<const uint8_t*>(in), reinterpret_cast<uint64_t*>(out), nbytes);
  return check_launch("bin_unpack");
}

extern "C" int nes_bin_sample_bits(const uint16_t* p_half, const float* uniforms, void* out, int64_t n,
                                   int64_t rows, int64_t cols, int word_bits, uint64_t seed,
                                   nes_stream_t stream) {
  NES_REQUIRE(n >= 0 && rows >= 0 && cols >= 0, NES_ERR_BAD_ARG, "bin_sample_bits: negative extent");
  NES_REQUIRE(word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "bin_sample_bits: word_bits must be 32 or 64");
  const int64_t row_u32 = ceil_div<int64_t>(cols, word_bits) * (word_bits / 32);
  const int64_t total = n * rows * row_u32;
  if (total == 0) return NES_OK;
  NES_REQUIRE(p_half && out, NES_ERR_BAD_ARG, "bin_sample_bits: null pointer");
  NES_REQUIRE(ceil_div<int64_t>(total, 256) <= INT32_MAX, NES_ERR_UNSUPPORTED, "bin_sample_bits: too large");
  NES_REQUIRE(rows <= UINT32_MAX && n <= UINT32_MAX, NES_ERR_UNSUPPORTED, "bin_sample_bits: too large");
  const __half* p = reinterpret_cast<const __half*>(p_half);
  const unsigned blocks = (unsigned)ceil_div<int64_t>(total, 256);
  if (uniforms) {
    const int vec = (cols % 4 == 0) && aligned16(uniforms) && ((reinterpret_cast<uintptr_t>(p_half) & 7u) == 0);
    sample_bits_kernel<<<blocks, 256, 0, as_stream(stream)>>>(p, uniforms, static_cast<uint32_t*>(out), n, rows, cols, row_u32, seed, vec);
  } else {
    const int64_t pairs = rows * row_u32;
    const int members = sample_members_per_block(n, ceil_div<int64_t>(pairs, 256));
    NES_REQUIRE(ceil_div<int64_t>(n, members) <= 65535, NES_ERR_UNSUPPORTED, "bin_sample_bits: more than %d members", 65535 * members);
    dim3 grid((unsigned)ceil_div<int64_t>(pairs, 256), (unsigned)ceil_div<int64_t>(n, members));
    sample_bits_philox_kernel<<<grid, 256, 0, as_stream(stream)>>>(p, static_cast<uint32_t*>(out), n, rows, cols, row_u32, seed, members);
  }
  return check_launch("bin_sample_bits");
}

extern "C" int nes_bin_bmm(const void* A, const void* B, int32_t* C, int64_t P, int64_t M, int64_t K,
                           int64_t N, int word_bits, nes_stream_t stream) {
  return bin_bmm_common(A, B, nullptr, C, nullptr, P, M, K, N, word_bits, as_stream(stream), "bin_bmm");
}

extern "C" int nes_bin_bmm_act(const void* A, const void* B, const int32_t* thresh, uint8_t* C, int64_t P,
                               int64_t M, int64_t K, int64_t N, int word_bits, nes_stream_t stream) {
  NES_REQUIRE(thresh || P * M * N == 0, NES_ERR_BAD_ARG, "bin_bmm_act: null threshold");
  return bin_bmm_common(A, B, thresh, nullptr, C, P, M, K, N, word_bits, as_stream(stream), "bin_bmm_act");
}

extern "C" int nes_bin_im2col(const void* in, void* out, int64_t P, int H, int W, int Cw, int fx, int fy,
                              int px, int py, int sx, int sy, int word_bits, nes_stream_t stream) {
  NES_REQUIRE(word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "bin_im2col: word_bits must be 32 or 64");
  WindowA wa; int ho, wo;
  int rc = make_window(wa, in, P, H, W, Cw, fx, fy, px, py, sx, sy, ho, wo, "bin_im2col");
  if (rc != NES_OK) return rc;
  const int64_t total = P * wa.M * wa.K;
  if (total == 0) return NES_OK;
  NES_REQUIRE(in && out, NES_ERR_BAD_ARG, "bin_im2col: null pointer");
  NES_REQUIRE(ceil_div<int64_t>(total, 256) <= INT32_MAX, NES_ERR_UNSUPPORTED, "bin_im2col: too large");
  const unsigned blocks = (unsigned)ceil_div<int64_t>(total, 256);
  if (word_bits == 64) im2col_kernel<uint64_t><<<blocks, 256, 0, as_stream(stream)>>>(wa, static_cast<uint64_t*>(out), total);
  else im2col_kernel<uint32_t><<<blocks, 256, 0, as_stream(stream)>>>(wa, static_cast<uint32_t*>(out), total);
  return check_launch("bin_im2col");
}

extern "C" int nes_bin_conv(const void* in, const void* filter, const int32_t* thresh, int32_t* out_counts,
                            uint8_t* out_bool, int64_t P, int H, int W, int Cw, int N, int fx, int fy,
                            int px, int py, int sx, int sy, int word_bits, nes_stream_t stream) {
  NES_REQUIRE(word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "bin_conv: word_bits must be 32 or 64");
  NES_REQUIRE(N >= 0, NES_ERR_BAD_ARG, "bin_conv: negative extent");
  WindowA wa; int ho, wo;
  int rc = make_window(wa, in, P, H, W, Cw, fx, fy, px, py, sx, sy, ho, wo, "bin_conv");
  if (rc != NES_OK) return rc;
  if (P == 0 || N == 0) return NES_OK;
  NES_REQUIRE(in && filter && (thresh ? (void*)out_bool : (void*)out_counts), NES_ERR_BAD_ARG, "bin_conv: null pointer");
  if (word_bits == 64)
    return launch_bin_gemm<uint64_t>(wa, filter, thresh, out_counts, out_bool, P, wa.M, wa.K, N, as_stream(stream), "bin_conv");
  return launch_bin_gemm<uint32_t>(wa, filter, thresh, out_counts, out_bool, P, wa.M, wa.K, N, as_stream(stream), "bin_conv");
}

extern "C" int64_t nes_bin_weighted_sum_scratch_bytes(int64_t D, int64_t rows, int64_t words, int word_bits) {
  if (D <= 0 || rows <= 0 || words <= 0) return 0;
  const int64_t row_u32 = words * (word_bits / 32);
  const WsPlan p = plan_weighted_sum(D, rows, row_u32);
  return int64_t(p.splits) * rows * row_u32 * 32 * (int64_t)sizeof(float);
}

extern "C" int nes_bin_weighted_sum(const void* in, const uint16_t* w_half, uint16_t* out_half, int64_t D,
                                    int64_t rows, int64_t words, int64_t zbits, int word_bits,
                                    void* scratch, int64_t scratch_bytes, nes_stream_t stream) {
  return nes::bin_weighted_sum_impl(in, w_half, out_half, D, rows, words, zbits, word_bits, scratch, scratch_bytes, as_stream(stream));
}

int nes::bin_weighted_sum_impl(const void* in, const uint16_t* w_half, uint16_t* out_half, int64_t D,
                               int64_t rows, int64_t words, int64_t zbits, int word_bits,
                               void* scratch, int64_t scratch_bytes, cudaStream_t st) {
  NES_REQUIRE(D >= 0 && rows >= 0 && words >= 0 && zbits >= 0, NES_ERR_BAD_ARG, "bin_weighted_sum: negative extent");
  NES_REQUIRE(word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "bin_weighted_sum: word_bits must be 32 or 64");
  NES_REQUIRE(zbits <= words * word_bits, NES_ERR_BAD_ARG, "bin_weighted_sum: zbits exceeds the packed row");
  if (rows == 0 || zbits == 0) return NES_OK;
  NES_REQUIRE(out_half && (D == 0 || (in && w_half)), NES_ERR_BAD_ARG, "bin_weighted_sum: null pointer");
  if (D == 0) { cudaMemsetAsync(out_half, 0, rows * zbits * sizeof(uint16_t), st); return NES_OK; }
  const int64_t row_u32 = words * (word_bits / 32);
  const WsPlan p = plan_weighted_sum(D, rows, row_u32);
  const int64_t need = int64_t(p.splits) * rows * zbits * (int64_t)sizeof(float);
  NES_REQUIRE(scratch && scratch_bytes >= need, NES_ERR_SCRATCH, "bin_weighted_sum: scratch needs %lld bytes", (long long)need);
  NES_REQUIRE(rows <= 65535 && p.splits <= 65535, NES_ERR_UNSUPPORTED, "bin_weighted_sum: rows > 65535");
  dim3 grid((unsigned)p.bx, (unsigned)rows, (unsigned)p.splits);
  // the four-member path needs whole warps per member slot (and so per active column range)
  if (p.cols_per_block % 32 == 0 && row_u32 % 32 == 0)
    weighted_sum_kernel<true><<<grid, WS_THREADS, 0, st>>>(static_cast<const uint32_t*>(in), reinterpret_cast<const __half*>(w_half),
                                                           static_cast<float*>(scratch), D, rows, int(row_u32), zbits,
                                                           p.d_per_split, p.cols_per_block, p.slots);
  else
    weighted_sum_kernel<false><<<grid, WS_THREADS, 0, st>>>(static_cast<const uint32_t*>(in), reinterpret_cast<const __half*>(w_half),
                                                            static_cast<float*>(scratch), D, rows, int(row_u32), zbits,
                                                            p.d_per_split, p.cols_per_block, p.slots);
  int rc = check_launch("bin_weighted_sum");
  if (rc != NES_OK) return rc;
  const int64_t n = rows * zbits;
  weighted_sum_finish_kernel<<<(unsigned)ceil_div<int64_t>(n, 256), 256, 0, st>>>(
      static_cast<const float*>(scratch), reinterpret_cast<__half*>(out_half), p.splits, n);
  return check_launch("bin_weighted_sum(finish)");
}

extern "C" int nes_bin_maxpool2d(const void* in, void* out, int64_t P, int H, int W, int Cw, int fx, int fy,
                                 int px, int py, int sx, int sy, int word_bits, nes_stream_t stream) {
  NES_REQUIRE(word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "bin_maxpool2d: word_bits must be 32 or 64");
  WindowA wa; int ho, wo;
  int rc = make_window(wa, in, P, H, W, Cw, fx, fy, px, py, sx, sy, ho, wo, "bin_maxpool2d");
  if (rc != NES_OK) return rc;
  const int64_t total = P * ho * wo * Cw;
  if (total == 0) return NES_OK;
  NES_REQUIRE(in && out, NES_ERR_BAD_ARG, "bin_maxpool2d: null pointer");
  NES_REQUIRE(ceil_div<int64_t>(total, 256) <= INT32_MAX, NES_ERR_UNSUPPORTED, "bin_maxpool2d: too large");
  const unsigned blocks = (unsigned)ceil_div<int64_t>(total, 256);
  if (word_bits == 64)
    maxpool_kernel<uint64_t><<<blocks, 256, 0, as_stream(stream)>>>(static_cast<const uint64_t*>(in), static_cast<uint64_t*>(out), total, H, W, Cw, ho, wo, px, py, sx, sy);
  else
    maxpool_kernel<uint32_t><<<blocks, 256, 0, as_stream(stream)>>>(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), total, H, W, Cw, ho, wo, px, py, sx, sy);
  return check_launch("bin_maxpool2d");
}

extern "C" int nes_bin_seeded_bmv(const uint16_t* p_half, const void* B, int32_t* C, int64_t n, int64_t rows,
                                  int64_t cols, int word_bits, uint64_t seed, nes_stream_t stream) {
  NES_REQUIRE(n >= 0 && rows >= 0 && cols >= 0, NES_ERR_BAD_ARG, "bin_seeded_bmv: negative extent");
  NES_REQUIRE(word_bits == 32 || word_bits == 64, NES_ERR_BAD_ARG, "bin_seeded_bmv: word_bits must be 32 or 64");
  if (n == 0 || rows == 0) return NES_OK;
  NES_REQUIRE(p_half && B && C, NES_ERR_BAD_ARG, "bin_seeded_bmv: null pointer");
  const int64_t row_u32 = ceil_div<int64_t>(cols, word_bits) * (word_bits / 32);
  cudaStream_t st = as_stream(stream);
  cudaMemsetAsync(C, 0, n * rows * sizeof(int32_t), st);
  if (row_u32 == 0) return NES_OK;
  const int64_t pairs = rows * row_u32;
  const int members = sample_members_per_block(n, ceil_div<int64_t>(pairs, 256));
  NES_REQUIRE(ceil_div<int64_t>(n, members) <= 65535 && ceil_div<int64_t>(pairs, 256) <= INT32_MAX, NES_ERR_UNSUPPORTED,
              "bin_seeded_bmv: too large");
  NES_REQUIRE(rows <= UINT32_MAX && n <= UINT32_MAX, NES_ERR_UNSUPPORTED, "bin_seeded_bmv: too large");
  dim3 grid((unsigned)ceil_div<int64_t>(pairs, 256), (unsigned)ceil_div<int64_t>(n, members));
  seeded_bmv_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const __half*>(p_half), static_cast<const uint32_t*>(B), C, n, rows, cols, row_u32, seed, members);
  return check_launch("bin_seeded_bmv");
}
