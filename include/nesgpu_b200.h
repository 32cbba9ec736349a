/*
 * nesgpu_b200 -- C ABI of the B200 (sm_100a) population-batched perturbed-layer kernels.
 *
 * Every entry point:
 *   - takes plain DEVICE pointers and sizes (no framework types), all tensors contiguous;
 *   - launches on the CUDA stream it is given (a cudaStream_t passed as void*), never
 *     synchronises the device, never allocates or frees memory;
 *   - returns NES_OK (0) or a negative nes_status; nes_last_error() gives the detail.
 * Kernels that need workspace take a caller-owned `scratch` pointer; the matching
 * *_scratch_bytes() function says how much.
 *
 * The reference project (jamesal1/NESgpu) has no C ABI: its layers are PyTorch modules
 * (modules/base.py, modules/binary.py) over ATen library calls, cupy RawKernels
 * (extensions/src/*.cu launched by extensions/booleanOperations.py) and a pybind
 * extension (extensions/booleanOperations.cpp, booleanUtilities.cpp).  Each declaration
 * below names the reference code it replaces as file:line within that project.
 *
 * Index conventions shared by the fp32 entry points (modules/base.py:357,368,490 and
 * :377-378,504-505,584-585): batch row b = r * D + d for member d in [0, D) and repeat r in
 * [0, R); when `antithetic` is non-zero the perturbation of rows with r >= (R + 1) / 2 is
 * negated.  Noise tensors already carry their scale (modules/base.py:83,206).
 */
#ifndef NESGPU_B200_H
#define NESGPU_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NES_ABI_VERSION 1

typedef void* nes_stream_t; /* cudaStream_t */

enum nes_status {
  NES_OK = 0,
  NES_ERR_BAD_ARG = -1,      /* null pointer, negative extent, misaligned buffer            */
  NES_ERR_UNSUPPORTED = -2,  /* a size or option outside what the kernels implement          */
  NES_ERR_LAUNCH = -3,       /* the CUDA runtime rejected a launch (see nes_last_error)      */
  NES_ERR_TIMEOUT = -4,      /* a bounded device-side wait ran out                           */
  NES_ERR_SCRATCH = -5       /* scratch buffer missing or smaller than *_scratch_bytes()     */
};

int nes_abi_version(void);
const char* nes_status_string(int status);
/* Detail of the last failure on the calling thread ("" if none). */
const char* nes_last_error(void);
/* Kernel launches issued by this library in the calling process so far (diagnostic counter; it has
 * no counterpart in the reference). */
int64_t nes_launch_count(void);

/* ------------------------------------------------------------------ fp32: plain layers */

/* y[M,N] = x[M,K] . weight[N,K]^T + bias[N] (bias may be NULL).
 * Replaces F.linear at modules/base.py:366,381,488. */
int nes_linear_fwd(const float* x, const float* weight, const float* bias, float* y,
                   int64_t M, int64_t N, int64_t K, nes_stream_t stream);

/* The same product on the tensor cores (TMA-fed tcgen05.mma, kind::tf32, fp32 accumulation in tensor
 * memory).  mode 1: operands rounded to TF32 (relative error ~1e-3; for callers that state it);
 * mode 3: error-compensated 3xTF32 (operands split into tf32 hi + lo parts, three products), fp32-level
 * accuracy.  K must be a multiple of 4.  `scratch` holds the rounded / split operand copies.
 * Replaces F.linear at modules/base.py:366,381,488. */
int64_t nes_linear_fwd_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int mode);
int nes_linear_fwd_tc(const float* x, const float* weight, const float* bias, float* y,
                      int64_t M, int64_t N, int64_t K, int mode,
                      void* scratch, int64_t scratch_bytes, nes_stream_t stream);
/* Reads (synchronously) the device words in which the tensor-core kernels record that one of their
 * bounded waits ran out (0 = none, 1 = producer, 2 = MMA issuer, 3 = epilogue, 4 = filter builder /
 * operand splitter) and clears them: a call reports what happened since the previous call.  A kernel whose
 * own wait ran out skips its stores, so its output is undefined; kernels launched afterwards are not
 * affected.  Call it where the host synchronises anyway (end of a step).  No counterpart in the reference. */
int nes_tc_error_flag(int* flag);

/* NCHW convolution, groups == 1, zero padding.  x (B,Cin,H,W), weight (Cout,Cin,kh,kw),
 * y (B,Cout,Ho,Wo).  Replaces F.conv2d at modules/base.py:411,558. */
int nes_conv2d_fwd(const float* x, const float* weight, const float* bias, float* y,
                   int64_t B, int Cin, int H, int W, int Cout, int kh, int kw,
                   int sh, int sw, int ph, int pw, int dh, int dw, nes_stream_t stream);

/* ------------------------------------------------- fp32: dense per-member (IID) noise */

/* PerturbedLinear.forward with the perturbed flag set (modules/base.py:355-381):
 *   y[b,o] = x[b].weight[o] + bias[o] + s(r) * (x[b].noise[d,o] + bias_noise[d,o]).
 * x (R*D,in), weight (out,in), noise (D,out,in), bias_noise (D,out) or NULL, y (R*D,out).
 * direct == 1 follows modules/base.py:356-364: noise holds W+E, bias_noise holds b+beta,
 * weight/bias are ignored and no sign is applied.  direct == 2: y already holds x.weight^T + bias
 * (for instance from nes_linear_fwd_tc) and only the per-member term is added to it. */
int nes_perturbed_linear_fwd(const float* x, const float* weight, const float* bias,
                             const float* noise, const float* bias_noise, float* y,
                             int64_t D, int64_t R, int64_t in, int64_t out,
                             int antithetic, int direct, nes_stream_t stream);

/* PerturbedConv2d.forward, non-direct branch (modules/base.py:410-425): per member a
 * convolution with weight + s(r)*noise[d] and bias + s(r)*bias_noise[d].
 * noise (D,Cout,Cin,kh,kw); bias/bias_noise may be NULL. */
int nes_perturbed_conv2d_fwd(const float* x, const float* weight, const float* bias,
                             const float* noise, const float* bias_noise, float* y,
                             int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                             int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                             int antithetic, nes_stream_t stream);

/* Perturbed.weight_grad plus the l1/l2 terms of Perturbed.update (modules/base.py:110-125):
 *   grad[i] = sum_d w[d] * noise[d,i] + l1 * sign(weight[i]) + l2 * weight[i],  i in [0,n).
 * `weight` may be NULL when l1 == l2 == 0.  Also used for the bias gradient
 * `weights @ bias_noise` (modules/base.py:135) with n = out.
 * The members are split over thread blocks; partial sums go through `scratch`. */
int64_t nes_perturbed_update_scratch_bytes(int64_t D, int64_t n);
int nes_perturbed_update(const float* noise, const float* w, const float* weight, float* grad,
                         int64_t D, int64_t n, float l1, float l2,
                         void* scratch, int64_t scratch_bytes, nes_stream_t stream);
/* The same reduction on a block of n columns of a wider noise matrix: member d's row starts at noise + d * ld
 * (ld >= n elements; ld == n is nes_perturbed_update).  Lets a caller form the gradient block by block, for
 * instance to hand finished blocks to an all-reduce while the next one streams.  weight / grad point at the
 * block's first element. */
int nes_perturbed_update_columns(const float* noise, const float* w, const float* weight, float* grad,
                                 int64_t D, int64_t n, int64_t ld, float l1, float l2,
                                 void* scratch, int64_t scratch_bytes, nes_stream_t stream);
/* The same reduction for "direct" storage (modules/base.py:111-117, 126-133), where the per-member
 * tensors hold parameter + noise:  grad[i] = sum_d w[d] * (stored[d,i] - param[i]) + l1/l2 terms.
 * The parameter is subtracted from each member's row before the row is weighted, as the reference does,
 * so the result does not lose digits to (sum_d w[d]) * param. */
int nes_perturbed_update_direct(const float* stored, const float* w, const float* param, const float* weight,
                                float* grad, int64_t D, int64_t n, float l1, float l2,
                                void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* nes_perturbed_update for callers that have no workspace to give.  (No counterpart in the
 * reference: there the reduction is one library GEMV that allocates whatever it likes.)
 *
 * Some hosts of this library own no device allocator of their own: a plug-in that is handed
 * input and output buffers by a runtime that owns all device memory, or a step that runs at a
 * point where the process must not create device memory.  They cannot size and provide the
 * `scratch` buffer of nes_perturbed_update, so this variant keeps the split partial sums in a
 * workspace built into the library: NES_NOALLOC_SCRATCH_FLOATS fp32 values (16 MiB) of device
 * memory that every GPU which loads the library holds until the process exits.  It performs no
 * cudaMalloc / cudaFree and calls no allocating routine.
 *
 *  - Limit: the call fails with NES_ERR_UNSUPPORTED (and says so in nes_last_error) when the
 *    member split needs more than the built-in workspace, i.e. when
 *    nes_perturbed_update_scratch_bytes(D, n) > 4 * NES_NOALLOC_SCRATCH_FLOATS
 *    (D = 1024, n = 1024*1024 is the largest benchmark shape that fits).
 *  - The first call on each device looks up the workspace address (with that device current);
 *    make that first call before any stream capture starts.
 *  - All calls on a device share the one workspace and it keeps the previous call's partial
 *    sums; every element that is read is rewritten first, so nothing has to start at zero --
 *    but two calls that overlap on the GPU (different streams, no ordering) race on it.
 *    Order them, or use nes_perturbed_update with separate buffers.
 * Arguments and result are those of nes_perturbed_update. */
#define NES_NOALLOC_SCRATCH_FLOATS 4194304
int nes_perturbed_update_noalloc(const float* noise, const float* w, const float* weight, float* grad,
                                 int64_t D, int64_t n, float l1, float l2, nes_stream_t stream);

/* Sparse Gaussian noise ("SparsePerturbedLinear", README.md:12,29-30; the layer has no
 * source in the reference snapshot): k (index,value) pairs per member and output row,
 *   y[b,o] = x[b].weight[o] + bias[o] + s(r) * (sum_t x[b, idx[d,o,t]] * val[d,o,t] + bias_noise[d,o]),
 * which equals PerturbedLinear.forward (modules/base.py:365-381) on the densified noise.
 * idx (D,out,k) int32 in [0,in); val (D,out,k). */
int nes_sparse_perturbed_linear_fwd(const float* x, const float* weight, const float* bias,
                                    const int32_t* idx, const float* val, const float* bias_noise,
                                    float* y, int64_t D, int64_t R, int64_t in, int64_t out,
                                    int k, int antithetic, nes_stream_t stream);

/* grad[o, idx[d,o,t]] += w[d] * val[d,o,t] over a zeroed grad, then + l1*sign(W) + l2*W:
 * Perturbed.update (modules/base.py:110-125) on the densified sparse noise. */
int nes_sparse_perturbed_update(const int32_t* idx, const float* val, const float* w,
                                const float* weight, float* grad, int64_t D, int64_t in,
                                int64_t out, int k, float l1, float l2, nes_stream_t stream);

/* The per-member term of nes_sparse_perturbed_linear_fwd on its own, added to a y that already holds
 * x.weight^T + bias (for instance from nes_linear_fwd_tc, which puts the base product on the tensor cores):
 *   y[b,o] += s(r) * (sum_t x[b, idx[d,o,t]] * val[d,o,t] + bias_noise[d,o]). */
int nes_sparse_noise_add(float* y, const float* x, const int32_t* idx, const float* val, const float* bias_noise,
                         int64_t D, int64_t R, int64_t in, int64_t out, int k, int antithetic, nes_stream_t stream);

/* ------------------------------------------- fp32: shared noise + member permutations */

/* Permuted.update for layers with output permutations only, in one launch (modules/base.py:261-266 scatter,
 * :513-518 / :590-599 product, :120-138 l1 / l2 and the bias gradient `weights @ bias_noise`):
 *   grad[k,m,t] = sum_s G[k,s] * eps[s,m,t] + l1 * sign(weight) + l2 * weight,
 *   G[k,s] = sum_d w[d] * [pout[d,k] == s and s < out_sp];   bias_grad[k] = sum_d w[d] * bias_noise[d,k].
 * bias_noise and bias_grad may both be NULL; weight may be NULL when l1 == l2 == 0.  No scratch memory. */
int nes_permuted_update_out(const float* eps, const float* w, const int16_t* pout, const float* weight,
                            const float* bias_noise, float* grad, float* bias_grad,
                            int64_t D, int in, int out, int out_sp, int ksize, float l1, float l2,
                            nes_stream_t stream);

/* PermutedLinear.forward, default branch (modules/base.py:487-508):
 *   xg[b,j] = x[b, pin[d,j]]            (j < in_sp; identity when pin == NULL)
 *   p[b,s]  = sum_j xg[b,j] * eps[s,j]  (s < out_sp)
 *   q[b,k]  = p[b, pout[d,k]] if pout[d,k] < out_sp else 0   (identity when pout == NULL)
 *   y[b,k]  = x[b].weight[k] + bias[k] + s(r) * (q[b,k] + bias_noise[d,k]).
 * eps (out_sp,in_sp); pin (D,in_sp) int16 or NULL; pout (D,out) int16 or NULL.
 * p goes through `scratch`. */
int64_t nes_permuted_linear_fwd_scratch_bytes(int64_t D, int64_t R, int64_t out_sp);
int nes_permuted_linear_fwd(const float* x, const float* weight, const float* bias,
                            const float* eps, const float* bias_noise,
                            const int16_t* pin, const int16_t* pout, float* y,
                            int64_t D, int64_t R, int64_t in, int64_t out,
                            int64_t in_sp, int64_t out_sp, int antithetic,
                            void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* The same layer without output permutations (pout == NULL) as ONE tensor-core product
 *   y = [ x | s(r) * xg ] . [ weight | eps ]^T + bias + s(r) * bias_noise[d]
 * (K = in + in_sp): a pre-pass writes the concatenated, TF32-rounded (mode 1), bf16 (mode 2; kind::f16
 * MMAs, relative error ~3e-3) or hi/lo-split operand (mode 3: tf32 parts, 3xTF32; mode 4: bf16 parts, three
 * kind::f16 products, half the operand bytes of mode 3; both at fp32-level accuracy) into `scratch`, then
 * the tcgen05 tile kernel of nes_linear_fwd_tc runs on it with the per-member bias term in its epilogue.  Rows of eps at or above out_sp count as zero.
 * Replaces the same reference lines (modules/base.py:487-508) for input-permuted layers. */
int64_t nes_permuted_linear_fwd_tc_scratch_bytes(int64_t D, int64_t R, int64_t in, int64_t out,
                                                 int64_t in_sp, int mode);
int nes_permuted_linear_fwd_tc(const float* x, const float* weight, const float* bias,
                               const float* eps, const float* bias_noise, const int16_t* pin,
                               float* y, int64_t D, int64_t R, int64_t in, int64_t out,
                               int64_t in_sp, int64_t out_sp, int antithetic, int mode,
                               void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* The same layer with output permutations only (pin == NULL, in_sp == in; pout may be NULL when
 * out_sp == out) as ONE tensor-core kernel and one launch: a thread-block cluster per tile of 128 batch
 * rows multiplies the rows by the stacked matrix [weight; eps] (tcgen05.mma kind::tf32, both accumulators
 * in tensor memory, operands brought in by TMA and split into tf32 hi + lo parts in shared memory), and
 * the epilogue gathers p[b, pout[d,k]] from the cluster's shared memory, applies s(r), adds bias_noise,
 * bias and the base product and stores y.  No scratch memory.  mode 3: 3xTF32, fp32-level accuracy;
 * mode 1: operands rounded to TF32 (relative error ~1e-3; for callers that state it).
 * nes_permuted_linear_out_fwd_tc_supported returns 1 when the shape is covered (in a positive multiple
 * of 4, out + out_sp <= 2048, out <= 32767), else 0; x, weight and eps must be 16-byte aligned.
 * Replaces F.linear + apply_output_permutation + the adds at modules/base.py:487-508,236-240. */
int nes_permuted_linear_out_fwd_tc_supported(int64_t D, int64_t R, int64_t in, int64_t out, int64_t out_sp, int mode);
int nes_permuted_linear_out_fwd_tc(const float* x, const float* weight, const float* bias,
                                   const float* eps, const float* bias_noise, const int16_t* pout,
                                   float* y, int64_t D, int64_t R, int64_t in, int64_t out, int64_t out_sp,
                                   int antithetic, int mode, nes_stream_t stream);

/* Out-permuted convolution of an input shared by all members, fused with ReLU and 2x2/2 max-pooling
 * (floor mode).  z (R, Cout + out_sp, Ho, Wo) is the plain convolution of the R shared images with
 * the stacked filter [weight; eps] and no bias (for instance from nes_conv2d_fwd); for b = r*D + d
 *   y[b, py, px, c] = relu(max_{2x2}( z[r, c] + s(r) * z[r, Cout + pout[d,c]] ) + bias[c] + s(r) * bias_noise[d,c])
 * with the noise term dropped where pout[d,c] >= out_sp (pout == NULL: identity).  y is channels-last,
 * (R*D, Ho/2, Wo/2, Cout); out_mode 0 stores fp32, 1 fp32 rounded to TF32, 2 bf16 (for a tensor-core
 * consumer), 3 bf16 with images 2q and 2q+1 interleaved by pixel, (R*D/2, Ho/2, Wo/2, 2, Cout), the input
 * layout of nes_permuted_conv_pool_fwd_bf16x2 (D even).
 * Replaces, for this case, PermutedConv2d.forward (modules/base.py:557-588) followed by the ReLU and
 * MaxPool2d modules of the reference's models (models/mnistmodels.py:35-57). */
int nes_shared_conv_pool_fwd(const float* z, const float* bias, const float* bias_noise,
                             const int16_t* pout, void* y, int64_t R, int64_t D, int Cout, int out_sp,
                             int Ho, int Wo, int antithetic, int out_mode, nes_stream_t stream);

/* Out-permuted convolution (no input permutations; stride 1, no padding, no dilation) fused with ReLU
 * and 2x2/2 max-pooling on the tensor cores (tcgen05, kind::tf32: operands rounded / truncated to
 * TF32, fp32 accumulation; a stated reduced-precision mode, relative error ~1e-3).
 * x_nhwc (R*D, H, W, 32) channels-last fp32; weight (Cout,32,kh,kw); eps (out_sp,32,kh,kw);
 * pout (D,Cout) or NULL; y (R*D, Cout, Ho/2, Wo/2) NCHW:
 *   y[b,c] = relu(maxpool2(conv(x[b], weight)[c] + s(r) * conv(x[b], eps)[pout[d,c]]) + bias[c] + s(r) * bias_noise[d,c]).
 * Covered: Cin == 32, Cout <= 64, out_sp <= 64, kh*kw <= 9, (2*(Ho/2)-1)*W + 2*(Wo/2) <= 128;
 * anything else returns NES_ERR_UNSUPPORTED.  `scratch` holds the stacked TF32 filter [W; eps].
 * Replaces, for this case, PermutedConv2d.forward (modules/base.py:557-588) followed by the ReLU and
 * MaxPool2d modules of the reference's models (models/mnistmodels.py:35-57). */
int64_t nes_permuted_conv_pool_fwd_tc_scratch_bytes(int kh, int kw);
int nes_permuted_conv_pool_fwd_tc(const float* x_nhwc, const float* weight, const float* bias,
                                  const float* eps, const float* bias_noise, const int16_t* pout,
                                  float* y, int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                  int kh, int kw, int out_sp, int antithetic,
                                  void* scratch, int64_t scratch_bytes, nes_stream_t stream);
/* The same kernel with bf16 operands (x_nhwc_bf16 (R*D, H, W, 32) bf16; the filter is rounded to bf16;
 * fp32 accumulation and fp32 y; relative error ~3e-3, the other stated reduced-precision mode): half the
 * MMA instructions and half the input bytes.  Scratch as for the TF32 form. */
int nes_permuted_conv_pool_fwd_bf16(const void* x_nhwc_bf16, const float* weight, const float* bias,
                                    const float* eps, const float* bias_noise, const int16_t* pout,
                                    float* y, int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                    int kh, int kw, int out_sp, int antithetic,
                                    void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* The bf16 form with TWO images per MMA (N = 256; such an MMA takes hardly longer than one with N = 128).
 * x_pairs_bf16 (R*D/2, H, W, 2, 32) bf16: images 2q and 2q+1 interleaved by pixel (out_mode 3 of
 * nes_shared_conv_pool_fwd).  Covered: Cin == 32, 13x13 images, 3x3 filters, Cout <= 64, R*D even.
 * y, scratch and everything else as for nes_permuted_conv_pool_fwd_bf16. */
/* The split form of the bf16 kernel, which holds the fp32 bar: the input comes as two bf16 tensors of the
 * same channels-last layout, x_hi = bf16(x) and x_lo = bf16(x - x_hi) (what nes_shared_conv_pool_fwd stores with
 * out_mode 4), the stacked filter is split the same way inside, and the accumulator takes
 * F_hi.x_hi + F_lo.x_hi + F_hi.x_lo: relative error a few 1e-6.  Same coverage as the bf16 kernel. */
int64_t nes_permuted_conv_pool_fwd_bf16x3_scratch_bytes(int kh, int kw);
int nes_permuted_conv_pool_fwd_bf16x3(const void* x_hi_bf16, const void* x_lo_bf16, const float* weight, const float* bias,
                                      const float* eps, const float* bias_noise, const int16_t* pout, float* y,
                                      int64_t D, int64_t R, int Cin, int H, int W, int Cout, int kh, int kw,
                                      int out_sp, int antithetic, void* scratch, int64_t scratch_bytes,
                                      nes_stream_t stream);
int nes_permuted_conv_pool_fwd_bf16x2(const void* x_pairs_bf16, const float* weight, const float* bias,
                                      const float* eps, const float* bias_noise, const int16_t* pout,
                                      float* y, int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                      int kh, int kw, int out_sp, int antithetic,
                                      void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* PermutedConv2d.forward, default branch (modules/base.py:557-588), evaluated as one
 * convolution per member with the effective filter
 *   W_d[k,c,:,:] = weight[k,c] + s(r) * eps[pout[d,k], j]  for the j with pin[d,j] == c
 * (zero where pout[d,k] >= out_sp or no such j), which is algebraically the same sum.
 * pin must not repeat a channel within a member (allow_repeats is handled by the caller
 * through nes_permuted_dense_noise + nes_perturbed_conv2d_fwd).
 * eps (out_sp,in_sp,kh,kw).  `scratch` holds the per-member channel maps. */
int64_t nes_permuted_conv2d_fwd_scratch_bytes(int64_t D, int Cin, int Cout);
int nes_permuted_conv2d_fwd(const float* x, const float* weight, const float* bias,
                            const float* eps, const float* bias_noise,
                            const int16_t* pin, const int16_t* pout, float* y,
                            int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                            int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                            int in_sp, int out_sp, int antithetic,
                            void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* Tensor-core (TF32) versions of the two per-member convolutions: same arguments and meaning as
 * nes_perturbed_conv2d_fwd / nes_permuted_conv2d_fwd (modules/base.py:410-425, 557-588), evaluated by a
 * persistent tcgen05 kernel that builds each member's effective filter in shared memory and reads the
 * input through TMA from a zero-padded channels-last TF32-rounded copy kept in `scratch`.  Reduced precision
 * (operands rounded to TF32, relative error ~1e-3): for callers that state it.  Supported: stride 1,
 * Cin % 32 == 0, Cout % 32 == 0 and <= 256, member filter <= ~200 KB, D*R <= 65535 images per call;
 * anything else returns NES_ERR_UNSUPPORTED. */
int64_t nes_conv2d_fwd_tc_scratch_bytes(int64_t D, int64_t R, int Cin, int H, int W, int Cout, int kh, int kw,
                                        int ph, int pw);
int nes_perturbed_conv2d_fwd_tc(const float* x, const float* weight, const float* bias,
                                const float* noise, const float* bias_noise, float* y,
                                int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                int antithetic, void* scratch, int64_t scratch_bytes, nes_stream_t stream);
int nes_permuted_conv2d_fwd_tc(const float* x, const float* weight, const float* bias,
                               const float* eps, const float* bias_noise,
                               const int16_t* pin, const int16_t* pout, float* y,
                               int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                               int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                               int in_sp, int out_sp, int antithetic,
                               void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* BF16 tensor-core versions (same arguments again): operands rounded to bf16, fp32 accumulation, the member
 * filter as the M operand (M = 64 / 128) and 256 output positions as N, so one tcgen05.mma does four times
 * the work of the TF32 path.  Reduced precision (relative error ~3e-3): for callers that state it.
 * Supported: stride 1, Cin % 64 == 0, Cout % 8 == 0 and <= 128, D*R <= 65535 images per call. */
int64_t nes_conv2d_fwd_bf16_scratch_bytes(int64_t D, int64_t R, int Cin, int H, int W, int Cout, int kh, int kw,
                                          int ph, int pw);
int nes_perturbed_conv2d_fwd_bf16(const float* x, const float* weight, const float* bias,
                                  const float* noise, const float* bias_noise, float* y,
                                  int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                  int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                  int antithetic, void* scratch, int64_t scratch_bytes, nes_stream_t stream);
int nes_permuted_conv2d_fwd_bf16(const float* x, const float* weight, const float* bias,
                                 const float* eps, const float* bias_noise,
                                 const int16_t* pin, const int16_t* pout, float* y,
                                 int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                 int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                 int in_sp, int out_sp, int antithetic,
                                 void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* The same kernels in their split form, which holds the fp32 bar on the tensor cores: filter and input are
 * each split into two bf16 parts (v = hi + lo + O(2^-18 |v|)) and the fp32 accumulator takes
 * W_hi.x_hi + W_lo.x_hi + W_hi.x_lo; relative error a few 1e-6.  Tiles are 128 positions; scratch holds two
 * staged copies of x.  nes_conv2d_fwd_bf16x3_supported returns 1 when the geometry is covered (stride 1,
 * Cin % 64 == 0, Cout % 8 == 0 and <= 128, dilation <= 8, both filter copies plus two input slots within
 * shared memory), else 0.  Replaces the same reference lines as the fp32 entry points
 * (modules/base.py:410-425, 557-588). */
int nes_conv2d_fwd_bf16x3_supported(int Cin, int H, int W, int Cout, int kh, int kw, int sh, int sw,
                                    int ph, int pw, int dh, int dw);
/* The same question for a permuted-noise layer (nes_permuted_conv2d_fwd_bf16x3): output-permuted layers with 64 input
 * channels, at most 64 output channels and at most 9 taps keep the member filter in tensor memory, which covers
 * larger images than the shared-memory form. */
int nes_permuted_conv2d_fwd_bf16x3_supported(int Cin, int H, int W, int Cout, int kh, int kw, int sh, int sw,
                                             int ph, int pw, int dh, int dw, int in_sp, int out_sp,
                                             int input_permutations);
int64_t nes_conv2d_fwd_bf16x3_scratch_bytes(int64_t D, int64_t R, int Cin, int H, int W, int Cout, int kh, int kw,
                                            int ph, int pw);
int nes_perturbed_conv2d_fwd_bf16x3(const float* x, const float* weight, const float* bias,
                                    const float* noise, const float* bias_noise, float* y,
                                    int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                    int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                    int antithetic, void* scratch, int64_t scratch_bytes, nes_stream_t stream);
int nes_permuted_conv2d_fwd_bf16x3(const float* x, const float* weight, const float* bias,
                                   const float* eps, const float* bias_noise,
                                   const int16_t* pin, const int16_t* pout, float* y,
                                   int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                                   int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                                   int in_sp, int out_sp, int antithetic,
                                   void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* The dense noise a Permuted layer is equal to (derived from modules/base.py:487-508):
 *   E[d,k,m,t] = sum_j [pin[d,j] == m] * eps[pout[d,k], j, t]   (0 where pout[d,k] >= out_sp).
 * E (D,out,in,ksize) is fully overwritten.  Repeated pin entries add. */
int nes_permuted_dense_noise(const float* eps, const int16_t* pin, const int16_t* pout, float* E,
                             int64_t D, int in, int out, int in_sp, int out_sp, int ksize,
                             nes_stream_t stream);

/* Permuted.get_permutation_weights + PermutedLinear/PermutedConv2d.weight_grad
 * (modules/base.py:242-267, 511-518, 590-599) plus the l1/l2 terms of update (:122-125):
 *   out-only: G[k,s] = sum_d w_d [pout[d,k] == s];  grad[k,m,t] = sum_s G[k,s] eps[s,m,t]
 *   in-only:  H[j,m] = sum_d w_d [pin[d,j] == m];   grad[k,m,t] = sum_j eps[k,j,t] H[j,m]
 *   both:     grad = sum_d w_d E_d  with E_d as in nes_permuted_dense_noise.
 * grad (out,in,ksize); ksize = kh*kw (1 for linear).  `perm_weights_out`, if not NULL,
 * receives G (out,out_sp) or H (in_sp,in) for the single-sided modes. */
int64_t nes_permuted_update_scratch_bytes(int in, int out, int in_sp, int out_sp);
int nes_permuted_update(const float* eps, const float* w, const int16_t* pin, const int16_t* pout,
                        const float* weight, float* grad, float* perm_weights_out,
                        int64_t D, int in, int out, int in_sp, int out_sp, int ksize,
                        float l1, float l2, void* scratch, int64_t scratch_bytes,
                        nes_stream_t stream);

/* PerturbedAffine.forward (modules/base.py:437-444): y[i] = x[i] * scale[i % period] + shift[i % period], the
 * (per-member) scale and shift tensors of `period` elements broadcast over the leading dimensions of x. */
int nes_affine_fwd(const float* x, const float* scale, const float* shift, float* y, int64_t n, int64_t period,
                   nes_stream_t stream);

/* ----------------------------------------------- fp32: shared noise + member sign flips */

/* SyntheticLinear.forward (modules/base.py:611-628):
 *   p[b,k] = sum_m x[b,m] * fin[d,m] * eps[k,m];  y[b,k] = x[b].weight[k] + bias[k] + s(r) * (p[b,k] * fout[d,k] + bias_noise[d,k]).
 * eps (out,in); fin (D,in) / fout (D,out) are +-1 int8, either may be NULL (= +1).  p goes through `scratch`. */
int64_t nes_synthetic_linear_fwd_scratch_bytes(int64_t D, int64_t R, int64_t out);
int nes_synthetic_linear_fwd(const float* x, const float* weight, const float* bias,
                             const float* eps, const float* bias_noise,
                             const int8_t* fin, const int8_t* fout, float* y,
                             int64_t D, int64_t R, int64_t in, int64_t out, int antithetic,
                             void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* The same layer with both products on the tensor cores (tcgen05 kind::tf32 on operands split into tf32
 * hi + lo parts; mode 3: 3xTF32, fp32-level accuracy; mode 1: plain TF32, for callers that state it):
 * y = x.weight^T + bias, p = (x * fin).eps^T, then one pass adds s(r) * (fout * p + bias_noise).  in must be
 * a multiple of 4.  scratch holds the split operands and p. */
int64_t nes_synthetic_linear_fwd_tc_scratch_bytes(int64_t D, int64_t R, int64_t in, int64_t out, int mode);
int nes_synthetic_linear_fwd_tc(const float* x, const float* weight, const float* bias, const float* eps,
                                const float* bias_noise, const int8_t* fin, const int8_t* fout, float* y,
                                int64_t D, int64_t R, int64_t in, int64_t out, int antithetic, int mode,
                                void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* SyntheticConv2d.forward (modules/base.py:642-668), evaluated as one convolution per member with the
 * effective filter W[k,c] + s(r) * fout[d,k] * fin[d,c] * eps[k,c]. */
int nes_synthetic_conv2d_fwd(const float* x, const float* weight, const float* bias,
                             const float* eps, const float* bias_noise,
                             const int8_t* fin, const int8_t* fout, float* y,
                             int64_t D, int64_t R, int Cin, int H, int W, int Cout,
                             int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                             int antithetic, nes_stream_t stream);

/* Synthetic.weight_grad (modules/base.py:338-347) plus the l1/l2 terms of update:
 *   grad[k,m,t] = eps[k,m,t] * sum_d w_d * fout[d,k] * fin[d,m]   (a missing side counts as +1).
 * For two-sided flips the reference's einsum multiplies by w_d twice (modules/base.py:340); this
 * entry point computes the fitness-weighted sum sum_d w_d E_d, which is what the one-sided branches do.
 * With one flipped side the flip weights are summed once into `scratch` (max(in, out) floats) and eps is
 * scaled by them; without scratch, and for two-sided flips, every gradient entry walks the members. */
int64_t nes_synthetic_update_scratch_bytes(int in, int out);
int nes_synthetic_update(const float* eps, const float* w, const int8_t* fin, const int8_t* fout,
                         const float* weight, float* grad, int64_t D, int in, int out, int ksize,
                         float l1, float l2, void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* ---------------------------------------------------------------- noise set-up (device) */

/* out[i] = mean + std * N(0,1), Philox-4x32-10 keyed by (seed, offset + i/4).
 * Replaces Tensor.normal_ at modules/base.py:83-85,206-208. */
int nes_fill_normal(float* out, int64_t n, float mean, float std, uint64_t seed, uint64_t offset,
                    nes_stream_t stream);
/* out[i] = lo + (hi - lo) * U(0,1].  Replaces torch.rand at modules/binary.py:63. */
int nes_fill_uniform(float* out, int64_t n, float lo, float hi, uint64_t seed, uint64_t offset,
                     nes_stream_t stream);
/* out[i] = +1 or -1 with equal probability (int8).  Replaces 2*randint(2)-1 at modules/base.py:323-328. */
int nes_fill_signs(int8_t* out, int64_t n, uint64_t seed, uint64_t offset, nes_stream_t stream);
/* D independent uniform permutations of [0,n), first `keep` entries of each stored
 * (out is (D,keep) int16); with_replacement != 0 draws keep independent indices instead.
 * Replaces the per-member CPU randperm loop / randint at modules/base.py:209-227.  n <= 16384
 * without replacement (the sort runs in shared memory), n <= 32767 with replacement.  Row i is the draw
 * of member first_member + i: a rank that owns members [lo, hi) of a population passes first_member = lo
 * and gets rows lo..hi-1 of the table a single process would draw with the same seed. */
int nes_sample_permutations(int16_t* out, int64_t D, int n, int keep, int with_replacement,
                            uint64_t seed, int64_t first_member, nes_stream_t stream);

/* ---------------------------------------------------------------------- bit-packed ops
 * word_bits is 64 (int64 words) or 32 (int32 words), as the reference's KernelWrapper
 * substitutes (extensions/booleanOperations.py:10-36).  bool tensors are one byte per value. */

/* (rows,cols) bool -> (rows, ceil(cols/word_bits)) words, LSB first.
 * Replaces pack_kernel (extensions/src/pack.cu:4-30) and cuda_pack (booleanUtilitiesCuda.cu:54-74,163-177). */
int nes_bin_pack(const uint8_t* in, void* out, int64_t rows, int64_t cols, int word_bits,
                 nes_stream_t stream);
/* (rows,cols) uint8 -> words, byte i -> bits 8i..8i+7.  Replaces int8pack_kernel (extensions/src/int8pack.cu:4-30). */
int nes_bin_int8pack(const uint8_t* in, void* out, int64_t rows, int64_t cols, int word_bits,
                     nes_stream_t stream);
/* (rows,cols) bool -> (rows, ceil(cols/8)) int8.  Replaces cuda_pack8 (booleanUtilitiesCuda.cu:31-50,148-158). */
int nes_bin_pack8(const uint8_t* in, int8_t* out, int64_t rows, int64_t cols, nes_stream_t stream);
/* (rows,words) words -> (rows, words*word_bits) bool.  Replaces cuda_unpack (booleanUtilitiesCuda.cu:77-90,182-195). */
int nes_bin_unpack(const void* in, uint8_t* out, int64_t rows, int64_t words, int word_bits,
                   nes_stream_t stream);

/* out[x,y,z] bit i = float(p[y, word_bits*z + i]) > u, for x in [0,n): Bernoulli(p) bits.
 * p (rows,cols) fp16.  If `uniforms` (n,rows,cols) fp32 is given it supplies u; otherwise a bit is
 * set when a 16-bit uniform integer from Philox-4x32-10 keyed by (seed, x, y, column) is below
 * ceil(p * 65536): Bernoulli(p) with p rounded up to a multiple of 2^-16.  The compare runs
 * bit-sliced over the 32 columns of a word (threshold bit-planes against random words, eight
 * random words per output word; a uniform's low byte reuses, rotated, bits that are high-byte
 * bits of other columns, so each uniform is sixteen independent bits).
 * Replaces sample_bits_kernel (extensions/src/sample_bits.cu:9-60) and cuda_sample_bits
 * (booleanUtilitiesCuda.cu:95-122,199-223). */
int nes_bin_sample_bits(const uint16_t* p_half, const float* uniforms, void* out, int64_t n,
                        int64_t rows, int64_t cols, int word_bits, uint64_t seed,
                        nes_stream_t stream);

/* Fused Bernoulli sampling + product: C[x,y] = sum_z popcount(bits(x,y,z) ^ B[x,z]) where bits(x,y,z) are
 * exactly the words nes_bin_sample_bits (device generator, same seed) would store -- the (n,rows,words) weight
 * bits are never materialised.  p (rows,cols) fp16, B (n, words) packed inputs, C (n, rows) int32.
 * Replaces cuda_binary_seeded_bmv (extensions/booleanOperationsCuda.cu:172-202,301-322). */
int nes_bin_seeded_bmv(const uint16_t* p_half, const void* B, int32_t* C, int64_t n, int64_t rows,
                       int64_t cols, int word_bits, uint64_t seed, nes_stream_t stream);

/* C[z,x,y] = sum_k popcount(A[z,x,k] ^ B[z,k,y]) as int32.  A (P,M,K), B (P,K,N), C (P,M,N).
 * Replaces bmm_kernel (extensions/src/bmm.cu:5-58) and cuda_binary_bmm (booleanOperationsCuda.cu:33-100,206-238). */
int nes_bin_bmm(const void* A, const void* B, int32_t* C, int64_t P, int64_t M, int64_t K,
                int64_t N, int word_bits, nes_stream_t stream);
/* C[z,x,y] = 2*acc > thresh[z,y] as bool.  Replaces bmm_act_kernel (extensions/src/bmm_act.cu:5-63). */
int nes_bin_bmm_act(const void* A, const void* B, const int32_t* thresh, uint8_t* C, int64_t P,
                    int64_t M, int64_t K, int64_t N, int word_bits, nes_stream_t stream);

/* Packed NHWC (P,H,W,Cw) -> columns (P, h*w, fx*fy*Cw); out-of-bounds taps give the zero word.
 * Replaces batch_im2col_kernel (extensions/src/batch_im2col.cu:3-33) and cuda_batch_im2col
 * (booleanOperationsCuda.cu:121-168,243-291). */
int nes_bin_im2col(const void* in, void* out, int64_t P, int H, int W, int Cw, int fx, int fy,
                   int px, int py, int sx, int sy, int word_bits, nes_stream_t stream);
/* out[p,xo,yo,n] = sum over window taps and channel words of popcount(in ^ filter), without
 * materialising the columns.  filter (P, fx*fy*Cw, N).  thresh == NULL: int32 counts to
 * `out_counts`; otherwise 2*acc > thresh[p,n] as bool to `out_bool`.
 * Replaces booleanOperations.conv / conv_act (extensions/booleanOperations.py:162-172) and
 * cuda_binary_batch_conv2d (booleanOperationsCuda.cu:295-298). */
int nes_bin_conv(const void* in, const void* filter, const int32_t* thresh, int32_t* out_counts,
                 uint8_t* out_bool, int64_t P, int H, int W, int Cw, int N, int fx, int fy,
                 int px, int py, int sx, int sy, int word_bits, nes_stream_t stream);

/* out[y,z] = half(sum_d float(w[d]) * bit_d[y,z]), fp32 accumulation.  in (D,rows,words),
 * w (D) fp16, out (rows,zbits) fp16.  Members are split over thread blocks; the fp32
 * partial sums go through `scratch`.
 * Replaces weighted_sum_kernel (extensions/src/weighted_sum.cu:8-48) and
 * cuda_binary_weighted_sum (booleanUtilitiesCuda.cu:125-145,225-240). */
int64_t nes_bin_weighted_sum_scratch_bytes(int64_t D, int64_t rows, int64_t words, int word_bits);
int nes_bin_weighted_sum(const void* in, const uint16_t* w_half, uint16_t* out_half, int64_t D,
                         int64_t rows, int64_t words, int64_t zbits, int word_bits,
                         void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* Bitwise OR over the 2x2 window starting at (xo*sx-px, yo*sy-py) of packed NHWC input;
 * fx, fy only enter the output size, as in max_pool2d_kernel (extensions/src/max_pool2d.cu:3-36). */
int nes_bin_maxpool2d(const void* in, void* out, int64_t P, int H, int W, int Cw, int fx, int fy,
                      int px, int py, int sx, int sy, int word_bits, nes_stream_t stream);

/* ------------------------------------------------------- bit-packed layers (modules/binary.py)
 * fp16 tensors are passed as uint16_t pointers.  Every fp16 step rounds once, as the reference's tensor
 * ops do; sums over fp16 values accumulate in fp32. */

/* Binarized.set_noise, probabilities (modules/binary.py:59-60):
 *   p = half(sigmoid(float(half(half(w / half(half(mean|w|) + 1e-5)) * 5)))).  scratch_sum: one float. */
int nes_binarized_probabilities(const uint16_t* weight_half, uint16_t* p_half, float* scratch_sum, int64_t n,
                                nes_stream_t stream);
/* Binarized.set_noise, bias noise (modules/binary.py:63-64): half(half(u - 0.5) * 6), u uniform on the fp16
 * grid of [0, 1), from Philox keyed by (seed, offset + i / 4). */
int nes_binarized_bias_noise(uint16_t* out_half, int64_t n, uint64_t seed, uint64_t offset, nes_stream_t stream);

/* Binarized.update (modules/binary.py:67-77): w = half(fitness), w -= mean(w); grad (rows, zbits) fp16 =
 * weighted bit sum of noise_bits (D, rows, words) with w, then += l1 * sign(weight), += l2 * weight;
 * bias_grad (out_degree) = w @ bias_noise (D, out_degree).  bias_noise / bias_grad may both be NULL. */
int64_t nes_binarized_update_scratch_bytes(int64_t D, int64_t rows, int64_t words, int word_bits);
int nes_binarized_update(const void* noise_bits, const float* fitness, const uint16_t* weight_half,
                         const uint16_t* bias_noise_half, uint16_t* grad_half, uint16_t* bias_grad_half,
                         int64_t D, int64_t rows, int64_t words, int64_t zbits, int64_t out_degree, int word_bits,
                         float l1, float l2, void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* BinarizedLinear.forward (modules/binary.py:93-103) on packed inputs x_packed (D, words): one streaming pass
 * over weight_bits (D, out, words), act = 2 * popcount(w ^ x) - in_bits.  out_kind 0: act as int32 (D, out);
 * 1: bool bytes half(act) > half(bias + bias_noise) (+ half(mean over the members of half(act)) when
 * batch_norm); 2: the same bits packed along `out` into word_bits-wide words (D, ceil(out / word_bits)), the
 * form the next packed layer reads.  Rows must be whole 16-byte chunks (at most 32 of them), D <= 65535.
 * scratch is used by batch_norm only. */
int64_t nes_binarized_linear_fwd_scratch_bytes(int64_t D, int64_t out, int batch_norm);
int nes_binarized_linear_fwd(const void* weight_bits, const void* x_packed, const uint16_t* bias_half,
                             const uint16_t* bias_noise_half, void* out, int64_t D, int64_t out_f, int64_t words,
                             int in_bits, int word_bits, int out_kind, int batch_norm,
                             void* scratch, int64_t scratch_bytes, nes_stream_t stream);

/* Threshold epilogue of BinarizedConv2d.forward (modules/binary.py:147-155) on the counts (P, S, N) of
 * nes_bin_conv, S = h * w positions: act = 2 * counts - offset; bit = half(act) > half(bias + bias_noise
 * (+ half(mean over the member's positions of half(act)) when batch_norm)).  out_kind 0: act as int32 (out may
 * be counts itself); 1: bool bytes (P, S, N); 2: bits packed along N (packed NHWC for the next layer).
 * sums: P * N floats of scratch for batch_norm. */
int nes_binarized_conv_epilogue(const int32_t* counts, const uint16_t* bias_half, const uint16_t* bias_noise_half,
                                void* out, int64_t P, int64_t S, int64_t N, int offset, int word_bits,
                                int out_kind, int batch_norm, float* sums, nes_stream_t stream);
/* int32 thresholds of the reference's conv_act call (modules/binary.py:156-157):
 *   out[p, n] = int(half(bias[n] + bias_noise[p, n])) + offset  (truncation toward zero). */
int nes_binarized_int_threshold(const uint16_t* bias_half, const uint16_t* bias_noise_half, int32_t* out,
                                int64_t P, int64_t N, int offset, nes_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* NESGPU_B200_H */
