"""Bit-packed tensor ops on B200 kernels, with the call signatures of the reference's
``extensions/booleanOperations.py`` (NESgpu) and of its pybind modules ``boolop_cuda`` /
``boolutil_cuda``.  Inputs and outputs are contiguous CUDA torch tensors; packed tensors are
``torch.int64`` or ``torch.int32`` words (LSB first).  Launches go to the CUDA stream that is
current at call time.  There is no CPU path.
"""
import torch

from . import _cabi as C


def _bits(dtype):
    if dtype == torch.int64:
        return 64
    if dtype == torch.int32:
        return 32
    raise NotImplementedError("packed words must be torch.int64 or torch.int32")


def ceil_div(a, b):
    return (a + b - 1) // b


def _out_hw(input, filterx, filtery, padx, pady, stridex, stridey):
    h = (input.size(1) - filterx + 2 * padx) // stridex + 1
    w = (input.size(2) - filtery + 2 * pady) // stridey + 1
    return h, w


def pack(input, dtype=torch.int32):
    """(rows, cols) bool -> (rows, ceil(cols/bits)) words (reference booleanOperations.py:175-187)."""
    assert len(input.shape) == 2
    input = C.require_cuda(input, "input", torch.bool)
    bits = _bits(dtype)
    ret = torch.empty((input.size(0), ceil_div(input.size(1), bits)), dtype=dtype, device=input.device)
    C.call("nes_bin_pack", C.ptr(input), C.ptr(ret), input.size(0), input.size(1), bits, C.stream())
    return ret


def int8pack(input, dtype=torch.int32):
    """(rows, cols) uint8 -> words holding bits/8 bytes each (reference booleanOperations.py:189-201)."""
    assert len(input.shape) == 2
    input = C.require_cuda(input, "input", torch.uint8)
    bits = _bits(dtype)
    ret = torch.empty((input.size(0), ceil_div(input.size(1), bits // 8)), dtype=dtype, device=input.device)
    C.call("nes_bin_int8pack", C.ptr(input), C.ptr(ret), input.size(0), input.size(1), bits, C.stream())
    return ret


def pack8(input):
    """(rows, cols) bool -> (rows, ceil(cols/8)) int8 (reference booleanUtilities.cpp:15-18)."""
    assert len(input.shape) == 2
    input = C.require_cuda(input, "input", torch.bool)
    ret = torch.empty((input.size(0), ceil_div(input.size(1), 8)), dtype=torch.int8, device=input.device)
    C.call("nes_bin_pack8", C.ptr(input), C.ptr(ret), input.size(0), input.size(1), C.stream())
    return ret


def unpack(input):
    """(rows, words) int8/int32/int64 -> (rows, words*bits) bool (reference booleanUtilities.cpp:43-46)."""
    assert len(input.shape) == 2
    bits = 8 if input.dtype == torch.int8 else _bits(input.dtype)
    input = C.require_cuda(input, "input")
    ret = torch.empty((input.size(0), input.size(1) * bits), dtype=torch.bool, device=input.device)
    C.call("nes_bin_unpack", C.ptr(input), C.ptr(ret), input.size(0), input.size(1), bits, C.stream())
    return ret


def sample_bits(p, n, dtype, seed, uniforms=None):
    """n independent Bernoulli(p) bit matrices, packed: (n, rows, ceil(cols/bits)) (reference
    booleanOperations.py:203-215).  ``uniforms`` (n, rows, cols) fp32 injects the random numbers
    (bit = p > u); without it they come from Philox keyed by ``seed``."""
    assert len(p.shape) == 2
    p = C.require_cuda(p, "p", torch.float16)
    bits = _bits(dtype)
    ret = torch.empty((n, p.size(0), ceil_div(p.size(1), bits)), dtype=dtype, device=p.device)
    if uniforms is not None:
        uniforms = C.require_cuda(uniforms, "uniforms", torch.float32)
        assert tuple(uniforms.shape) == (n, p.size(0), p.size(1))
    C.call("nes_bin_sample_bits", C.ptr(p), C.ptr(uniforms), C.ptr(ret), n, p.size(0), p.size(1), bits,
           int(seed) & (2 ** 64 - 1), C.stream())
    return ret


def binary_seeded_bmv(A, B, seed):
    """Fused Bernoulli sampling + XOR-popcount product (reference pybind name ``boolop_cuda.binary_seeded_bmv``,
    booleanOperations.cpp:58-63): ``A`` (out, in) fp16 probabilities, ``B`` (batch, words) packed inputs ->
    (batch, out) int32, equal to ``bmm(sample_bits(A, batch, B.dtype, seed), B.view(batch, -1, 1))`` without
    storing the sampled bits."""
    assert len(A.shape) == 2 and len(B.shape) == 2
    A = C.require_cuda(A, "A", torch.float16)
    B = C.require_cuda(B, "B")
    bits = _bits(B.dtype)
    assert B.size(1) == ceil_div(A.size(1), bits)
    ret = torch.empty((B.size(0), A.size(0)), dtype=torch.int32, device=A.device)
    C.call("nes_bin_seeded_bmv", C.ptr(A), C.ptr(B), C.ptr(ret), B.size(0), A.size(0), A.size(1), bits,
           int(seed) & (2 ** 64 - 1), C.stream())
    return ret


def _bmm_args(A, B):
    assert len(A.shape) == 3
    assert len(B.shape) == 3
    assert A.size(0) == B.size(0)
    assert A.size(2) == B.size(1)
    assert A.dtype == B.dtype
    return C.require_cuda(A, "A"), C.require_cuda(B, "B"), _bits(A.dtype)


def bmm(A, B):
    """C[z,x,y] = sum_k popcount(A[z,x,k] ^ B[z,k,y]) as int32 (reference booleanOperations.py:107-129)."""
    A, B, bits = _bmm_args(A, B)
    ret = torch.empty((A.size(0), A.size(1), B.size(2)), dtype=torch.int32, device=A.device)
    C.call("nes_bin_bmm", C.ptr(A), C.ptr(B), C.ptr(ret), A.size(0), A.size(1), A.size(2), B.size(2), bits, C.stream())
    return ret


def bmm_act(A, B, threshold):
    """2 * bmm(A, B) > threshold[z, y] as bool (reference booleanOperations.py:131-158)."""
    A, B, bits = _bmm_args(A, B)
    assert len(threshold.shape) == 2
    assert A.size(0) == threshold.size(0)
    assert threshold.size(1) == B.size(2)
    assert threshold.dtype == torch.int32
    threshold = C.require_cuda(threshold, "threshold")
    ret = torch.empty((A.size(0), A.size(1), B.size(2)), dtype=torch.bool, device=A.device)
    C.call("nes_bin_bmm_act", C.ptr(A), C.ptr(B), C.ptr(threshold), C.ptr(ret), A.size(0), A.size(1), A.size(2),
           B.size(2), bits, C.stream())
    return ret


def batch_im2col(input, filterx, filtery, padx, pady, stridex, stridey, REPEAT=128):
    """Packed NHWC (P,H,W,Cw) -> (P, h*w, fx*fy*Cw) columns (reference booleanOperations.py:82-102).
    ``REPEAT`` was a launch-shape knob of the reference kernel and is accepted and ignored."""
    assert len(input.shape) == 4
    input = C.require_cuda(input, "input")
    bits = _bits(input.dtype)
    h, w = _out_hw(input, filterx, filtery, padx, pady, stridex, stridey)
    ret = torch.empty((input.size(0), h * w, filterx * filtery * input.size(3)), dtype=input.dtype, device=input.device)
    C.call("nes_bin_im2col", C.ptr(input), C.ptr(ret), input.size(0), input.size(1), input.size(2), input.size(3),
           filterx, filtery, padx, pady, stridex, stridey, bits, C.stream())
    return ret


def _conv(input, filter, threshold, filterx, filtery, padx, pady, stridex, stridey):
    assert len(input.shape) == 4 and len(filter.shape) == 3
    assert input.size(0) == filter.size(0)
    assert filter.size(1) == filterx * filtery * input.size(3)
    assert input.dtype == filter.dtype
    input = C.require_cuda(input, "input")
    filter = C.require_cuda(filter, "filter")
    bits = _bits(input.dtype)
    h, w = _out_hw(input, filterx, filtery, padx, pady, stridex, stridey)
    N = filter.size(2)
    counts = bools = None
    if threshold is None:
        counts = torch.empty((input.size(0), h, w, N), dtype=torch.int32, device=input.device)
    else:
        assert threshold.dtype == torch.int32 and tuple(threshold.shape) == (input.size(0), N)
        threshold = C.require_cuda(threshold, "threshold")
        bools = torch.empty((input.size(0), h, w, N), dtype=torch.bool, device=input.device)
    C.call("nes_bin_conv", C.ptr(input), C.ptr(filter), C.ptr(threshold), C.ptr(counts), C.ptr(bools),
           input.size(0), input.size(1), input.size(2), input.size(3), N, filterx, filtery, padx, pady,
           stridex, stridey, bits, C.stream())
    return counts if threshold is None else bools


def conv(input, filter, filterx, filtery, padx, pady, stridex, stridey):
    """XOR-popcount convolution of packed NHWC input with per-member filters (P, fx*fy*Cw, out) ->
    (P, h, w, out) int32 (reference booleanOperations.py:162-166), without materialising columns."""
    return _conv(input, filter, None, filterx, filtery, padx, pady, stridex, stridey)


def conv_act(input, filter, threshold, filterx, filtery, padx, pady, stridex, stridey):
    """2 * conv > threshold[p, out] as bool (reference booleanOperations.py:168-172)."""
    return _conv(input, filter, threshold, filterx, filtery, padx, pady, stridex, stridey)


def weighted_sum(input, weights, zbits):
    """(rows, zbits) fp16 = sum_d weights[d] * bit_d (reference booleanOperations.py:218-229)."""
    assert len(input.shape) == 3
    assert input.size(0) == weights.size(0)
    input = C.require_cuda(input, "input")
    weights = C.require_cuda(weights, "weights", torch.float16)
    bits = _bits(input.dtype)
    ret = torch.empty((input.size(1), zbits), dtype=torch.float16, device=input.device)
    nbytes = C.call("nes_bin_weighted_sum_scratch_bytes", input.size(0), input.size(1), input.size(2), bits)
    buf = C.scratch(nbytes, input.device)
    C.call("nes_bin_weighted_sum", C.ptr(input), C.ptr(weights), C.ptr(ret), input.size(0), input.size(1),
           input.size(2), zbits, bits, C.ptr(buf), nbytes, C.stream())
    return ret


def max_pool2d(input, filterx, filtery, padx, pady, stridex, stridey, REPEAT=128):
    """Bitwise OR over a 2x2 window of packed NHWC input (reference booleanOperations.py:232-252;
    as in the reference kernel the window is 2x2 whatever filterx/filtery, which only set the
    output size)."""
    assert len(input.shape) == 4
    input = C.require_cuda(input, "input")
    bits = _bits(input.dtype)
    h, w = _out_hw(input, filterx, filtery, padx, pady, stridex, stridey)
    ret = torch.empty((input.size(0), h, w, input.size(3)), dtype=input.dtype, device=input.device)
    C.call("nes_bin_maxpool2d", C.ptr(input), C.ptr(ret), input.size(0), input.size(1), input.size(2),
           input.size(3), filterx, filtery, padx, pady, stridex, stridey, bits, C.stream())
    return ret


# names of the reference's pybind modules (booleanOperations.cpp:86-94, booleanUtilities.cpp:61-67)
binary_bmm = bmm
binary_batch_conv2d = conv


def binary_weighted_sum(input, weights, z_bits):
    return weighted_sum(input, weights, z_bits)
