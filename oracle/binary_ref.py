"""CPU oracle for the bit-packed binary path.  TEST INFRASTRUCTURE ONLY.

numpy restatement of the integer arithmetic of the reference's CUDA kernels in
``extensions/src/*.cu`` and ``extensions/booleanUtilitiesCuda.cu`` and of the layer glue in
``modules/binary.py`` (NESgpu).  The reference has no CPU implementation of these (it needs
cupy and a GPU at import), so this port is also the timed CPU baseline for the binary
configuration.  Only tests, the smoke check and the benchmark's CPU-baseline leg may import
this file; the product never does.

Parity status: pinned against the reference's own naive formulas in ``booloptests.py``
(+-1 grouped convolution with -1 padding, lines 150-160; ``conv_act == 2*conv > thresh``,
lines 157-159; max-pool == ``F.max_pool2d`` on the unpacked bits, lines 94-95,138-141); the
stored vectors come from ``tests/golden/make_golden.py``.  Bernoulli sampling is defined
"given the same uniforms": the reference's XORWOW stream mapping (sample_bits.cu:23-25) is
not reproduced.
"""
import numpy as np


def _word_dtype(bits):
    if bits == 64:
        return np.uint64, np.int64
    if bits == 32:
        return np.uint32, np.int32
    raise NotImplementedError("word width must be 32 or 64")


def pack(bools, bits=64):
    """pack_kernel (extensions/src/pack.cu:21-28): bit i of word y of row x is
    in[x, bits*y + i] (LSB first); columns past the end read as 0 (pack.cu:17)."""
    u, s = _word_dtype(bits)
    b = np.asarray(bools).astype(bool)
    rows, cols = b.shape
    words = (cols + bits - 1) // bits
    padded = np.zeros((rows, words * bits), dtype=bool)
    padded[:, :cols] = b
    shifts = np.arange(bits, dtype=u)
    vals = (padded.reshape(rows, words, bits).astype(u) << shifts).sum(axis=2, dtype=u)
    return vals.view(s)


def unpack(words, bits=64):
    """cuda_unpack_kernel (extensions/booleanUtilitiesCuda.cu:77-90)."""
    u, _ = _word_dtype(bits)
    w = np.ascontiguousarray(words).view(u)
    shifts = np.arange(bits, dtype=u)
    return (((w[..., None] >> shifts) & u(1)) > 0).reshape(*w.shape[:-1], w.shape[-1] * bits)


def pack8(bools):
    """cuda_pack8_kernel (extensions/booleanUtilitiesCuda.cu:31-50): bool -> int8, LSB first."""
    b = np.asarray(bools).astype(bool)
    rows, cols = b.shape
    words = (cols + 7) // 8
    padded = np.zeros((rows, words * 8), dtype=np.uint8)
    padded[:, :cols] = b
    vals = (padded.reshape(rows, words, 8) << np.arange(8, dtype=np.uint8)).sum(axis=2, dtype=np.uint8)
    return vals.view(np.int8)


def int8pack(bytes_, bits=64):
    """int8pack_kernel (extensions/src/int8pack.cu:21-28): byte i of a word's group goes to
    bits 8i..8i+7; bytes past the end read as 0 (int8pack.cu:17)."""
    u, s = _word_dtype(bits)
    a = np.asarray(bytes_).astype(np.uint8)
    rows, cols = a.shape
    per = bits // 8
    words = (cols + per - 1) // per
    padded = np.zeros((rows, words * per), dtype=np.uint8)
    padded[:, :cols] = a
    shifts = (np.arange(per) * 8).astype(u)
    vals = (padded.reshape(rows, words, per).astype(u) << shifts).sum(axis=2, dtype=u)
    return vals.view(s)


def conv_out_size(size, f, p, s):
    """booleanOperations.py:83-84."""
    return (size - f + 2 * p) // s + 1


def batch_im2col(inp, fx, fy, px, py, sx, sy):
    """batch_im2col_kernel (extensions/src/batch_im2col.cu:14-29): packed NHWC (P,H,W,Cw) ->
    (P, h*w, fx*fy*Cw); element = (i*fy + j)*Cw + c; out-of-bounds taps are the zero word."""
    P, H, W, Cw = inp.shape
    h = conv_out_size(H, fx, px, sx)
    w = conv_out_size(W, fy, py, sy)
    out = np.zeros((P, h, w, fx, fy, Cw), dtype=inp.dtype)
    for i in range(fx):
        for j in range(fy):
            for xo in range(h):
                xi = i + xo * sx - px
                if xi < 0 or xi >= H:
                    continue
                yi = j + np.arange(w) * sy - py
                ok = (yi >= 0) & (yi < W)
                out[:, xo, ok, i, j, :] = inp[:, xi, yi[ok], :]
    return out.reshape(P, h * w, fx * fy * Cw)


def bmm(A, B):
    """bmm_kernel (extensions/src/bmm.cu:40,48-53): C[z,x,y] = sum_k popcount(A[z,x,k] ^ B[z,k,y])
    as int32 -- XOR, i.e. a Hamming distance."""
    u = np.uint64 if A.dtype.itemsize == 8 else np.uint32
    Au = np.ascontiguousarray(A).view(u)
    Bu = np.ascontiguousarray(B).view(u)
    P, M, K = Au.shape
    N = Bu.shape[2]
    C = np.zeros((P, M, N), dtype=np.int32)
    for k in range(K):
        C += np.bitwise_count(Au[:, :, k, None] ^ Bu[:, k, None, :]).astype(np.int32)
    return C


def bmm_act(A, B, thresh):
    """bmm_act_kernel (extensions/src/bmm_act.cu:56): 2*acc > thresh[z, y]."""
    return 2 * bmm(A, B) > np.asarray(thresh, dtype=np.int32)[:, None, :]


def conv(inp, filt, fx, fy, px, py, sx, sy):
    """booleanOperations.conv (extensions/booleanOperations.py:162-166): im2col then bmm,
    viewed as (P, h, w, out)."""
    h = conv_out_size(inp.shape[1], fx, px, sx)
    w = conv_out_size(inp.shape[2], fy, py, sy)
    return bmm(batch_im2col(inp, fx, fy, px, py, sx, sy), filt).reshape(inp.shape[0], h, w, -1)


def conv_act(inp, filt, thresh, fx, fy, px, py, sx, sy):
    """booleanOperations.conv_act (extensions/booleanOperations.py:168-172)."""
    h = conv_out_size(inp.shape[1], fx, px, sx)
    w = conv_out_size(inp.shape[2], fy, py, sy)
    return bmm_act(batch_im2col(inp, fx, fy, px, py, sx, sy), filt, thresh).reshape(
        inp.shape[0], h, w, -1)


def max_pool2d(inp, fx, fy, px, py, sx, sy):
    """max_pool2d_kernel (extensions/src/max_pool2d.cu:19-32): bitwise OR over a window that
    the kernel fixes at 2x2 whatever fx, fy say (they only enter the output size)."""
    P, H, W, Cw = inp.shape
    h = conv_out_size(H, fx, px, sx)
    w = conv_out_size(W, fy, py, sy)
    out = np.zeros((P, h, w, Cw), dtype=inp.dtype)
    for i in range(2):
        for j in range(2):
            for xo in range(h):
                xi = i + xo * sx - px
                if xi < 0 or xi >= H:
                    continue
                yi = j + np.arange(w) * sy - py
                ok = (yi >= 0) & (yi < W)
                out[:, xo, ok, :] |= inp[:, xi, yi[ok], :]
    return out


def sample_bits(p_half, uniforms, bits=64):
    """sample_bits_kernel (extensions/src/sample_bits.cu:35,51-57) with the uniforms injected:
    bit i of ret[x, y, z] = float(P[y, bits*z + i]) > u[x, y, bits*z + i]; padding columns use
    P = 0 and so give 0 bits."""
    p = np.asarray(p_half, dtype=np.float16).astype(np.float32)
    u = np.asarray(uniforms, dtype=np.float32)
    n = u.shape[0]
    out = []
    for x in range(n):
        out.append(pack(p > u[x], bits))
    return np.stack(out)


def weighted_sum(inp, weights_half, zbits):
    """weighted_sum_kernel (extensions/src/weighted_sum.cu:36-46): ret[y, z] =
    half(sum_d float(w[d]) * bit_d[y, z]) with an fp32 accumulator in member order."""
    bits = inp.dtype.itemsize * 8
    w = np.asarray(weights_half, dtype=np.float16).astype(np.float32)
    D, rows, _ = inp.shape
    acc = np.zeros((rows, zbits), dtype=np.float32)
    for d in range(D):
        b = unpack(inp[d], bits)[:, :zbits]
        acc += np.where(b, w[d], np.float32(0))
    return acc.astype(np.float16)


def bernoulli_probabilities(weight_half):
    """Binarized.set_noise (modules/binary.py:59-60): sigmoid(5 * W / (mean|W| + 1e-5)) as fp16,
    computed the way torch does it for an fp16 parameter (fp16 division and scaling, fp32 sigmoid)."""
    import torch
    w = torch.as_tensor(np.asarray(weight_half, dtype=np.float16))
    norm = w / (w.abs().mean() + 1e-5) * 5
    return torch.sigmoid(norm.float()).half().numpy()


def binarized_linear_forward(weight_bits, inputs_bool, in_features, threshold=None, bits=64):
    """BinarizedLinear.forward (modules/binary.py:93-103) without batch-norm: activation =
    2 * bmm(weight_bits, pack(x).view(D, -1, 1)) - in_features, optionally compared with a
    (D, out) threshold."""
    D = weight_bits.shape[0]
    xb = pack(inputs_bool, bits).reshape(D, -1, 1)
    act = 2 * bmm(weight_bits, xb)[:, :, 0] - in_features
    if threshold is None:
        return act
    return act > threshold


# ----------------------------------------------------------------------------------
# Layer glue of modules/binary.py with torch's fp16 semantics spelled out: every fp16 tensor
# op is computed in fp32 and rounded once to fp16; an int32 tensor compared with an fp16 tensor
# is first converted to fp16.
# ----------------------------------------------------------------------------------

def _h(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16)


def _f(x):
    return np.asarray(x, dtype=np.float16).astype(np.float32)


def threshold_bits(act, bias_half, bias_noise_half, mean_half=None):
    """``activation > thresh`` of modules/binary.py:98-102 and :150-153.  act (..., N) int32; bias (N,);
    bias_noise broadcastable to act; mean_half (optional) broadcastable to act."""
    th = _h(_f(bias_half) + _f(bias_noise_half))
    if mean_half is not None:
        th = _h(_f(th) + _f(mean_half))
    return np.asarray(act).astype(np.float16) > th


def binarized_linear_layer(weight_bits, inputs_bool, in_features, bias_half, bias_noise_half, batch_norm, bits=64):
    """BinarizedLinear.forward with threshold=True (modules/binary.py:93-103): the batch mean is taken over the
    members (dim 0) of the fp16 activation."""
    act = binarized_linear_forward(weight_bits, inputs_bool, in_features, None, bits)
    mean = None
    if batch_norm:
        mean = _h(_f(act.astype(np.float16)).sum(axis=0, keepdims=True, dtype=np.float32) / np.float32(act.shape[0]))
    return threshold_bits(act, bias_half, bias_noise_half, mean)


def binarized_conv_layer(counts, offset, bias_half, bias_noise_half, batch_norm):
    """BinarizedConv2d.forward with threshold=True (modules/binary.py:139-157) on the conv counts (P, h, w, N).
    batch_norm: fp16 compare against bias + bias_noise + mean over the member's positions; otherwise the
    integer compare ``2 * counts > int(bias + bias_noise) + offset`` of the conv_act call."""
    counts = np.asarray(counts, dtype=np.int64)
    P = counts.shape[0]
    if not batch_norm:
        th = _h(_f(bias_half) + _f(bias_noise_half)).astype(np.float32)
        thresh = np.trunc(th).astype(np.int64) + offset
        return 2 * counts > thresh.reshape(P, 1, 1, -1)
    act = (2 * counts - offset).astype(np.int32)
    a16 = _f(act.astype(np.float16))
    mean = _h(a16.sum(axis=(1, 2), dtype=np.float32) / np.float32(act.shape[1] * act.shape[2]))      # (P, N)
    th = _h(_f(_h(_f(bias_half) + _f(bias_noise_half))) + _f(mean))
    return act.astype(np.float16) > th.reshape(P, 1, 1, -1)


def binarized_update(weight_bits, fitness, weight_half, bias_noise_half, in_degree, l1=0.0, l2=1e-3):
    """Binarized.update (modules/binary.py:67-77).  Returns (weight grad fp16, bias grad fp16)."""
    w16 = _h(fitness)
    mean = _h(_f(w16).sum(dtype=np.float32) / np.float32(w16.size))
    w = _h(_f(w16) - _f(mean))
    grad = weighted_sum(weight_bits, w, in_degree)
    wf = _f(weight_half)
    if l1:
        grad = _h(_f(grad) + _f(_h(np.float32(l1) * np.sign(wf))))
    if l2:
        grad = _h(_f(grad) + _f(_h(np.float32(l2) * wf)))
    bias_grad = _h((_f(w)[:, None] * _f(bias_noise_half)).sum(axis=0, dtype=np.float32))
    return grad, bias_grad
