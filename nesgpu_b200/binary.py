"""Bit-packed population layers behind the reference's ``modules/binary.py`` interface (NESgpu).

Each member owns a weight matrix of +-1 values drawn as Bernoulli(sigmoid(5 W / mean|W|)) and
stored as packed bits ``(directions, out, ceil(in/bits))``; activations are bools / packed
bits; the product is an XOR-popcount.  The classes keep the reference's names, constructor
arguments and attributes; their methods only validate and launch -- probabilities, bias noise,
fitness centring, l1 / l2 terms, bias gradient, the ``2 * counts - n`` activation, the fp16
thresholds (with or without the batch mean) and the packing of the output bits all run in the
CUDA library (``csrc/binary_layers.cu``).  Only population mode exists, as in the reference
(``forward`` with the perturbed flag off raises).

One addition: ``layer.packed_output = True`` makes a thresholding layer return its bits already
packed into ``dtype`` words (``(directions, ceil(out/bits))`` for the linear layer, packed NHWC
for the convolution) -- the form the next binary layer takes without a ``pack`` call.
"""
import torch
from torch import nn
from torch.nn.parameter import Parameter

from . import _cabi as C
from . import boolean_operations as booleanOperations
from .base import Perturbed, PerturbedModel  # noqa: F401  (re-exported like the reference's star import)

_F16 = torch.float16


class AsType(nn.Module):
    def __init__(self, dtype):
        super().__init__()
        self.dtype = dtype

    def forward(self, x):
        return x.type(self.dtype)


class ExtractBits(nn.Module):
    """Integer tensor -> its bits along a new trailing axis, LSB first (reference binary.py:20-29)."""

    def __init__(self, dtype):
        super().__init__()
        self.dtype = dtype
        self.bitlength = torch.iinfo(dtype).bits
        self.mask = 2 ** torch.arange(self.bitlength, dtype=dtype)

    def forward(self, input):
        mask = self.mask.to(input.device)
        return (input.unsqueeze(-1) & mask).view(*input.shape[:-1], -1) > 0


def _word_bits(dtype):
    return booleanOperations._bits(dtype)


def _half_ptr(t, name):
    return C.ptr(C.require_cuda(t.detach(), name, _F16))


class Binarized(nn.Module, Perturbed):
    """State and noise / update launches shared by the binary layers (reference binary.py:32-77)."""

    def __init__(self, in_degree, out_degree, directions, threshold=False, dtype=torch.int64, device="cuda"):
        nn.Module.__init__(self)
        self.bias = None            # set by the subclass when it thresholds
        Perturbed.__init__(self, directions)
        self.in_degree = in_degree
        self.out_degree = out_degree
        self.dtype = dtype
        self.threshold = threshold
        self.device = device
        self.uniforms = None        # optional injected (directions, rows, cols) fp32 uniforms for set_noise
        self.packed_output = False

    def reset_parameters(self):
        with torch.no_grad():
            self.weight.zero_()
            if self.bias is not None:
                self.bias.zero_()

    def bernoulli_probabilities(self):
        """sigmoid(5 W / (mean|W| + 1e-5)) as fp16, every step rounded as the reference's fp16 tensor ops round
        (reference binary.py:59-60)."""
        w = C.require_cuda(self.weight.detach(), "weight", _F16)
        p = torch.empty_like(w)
        acc = torch.empty(1, device=w.device, dtype=torch.float32)
        C.call("nes_binarized_probabilities", C.ptr(w), C.ptr(p), C.ptr(acc), w.numel(), C.stream())
        return p

    def set_noise(self, noise_scale=None):
        """Per-member weight bits and bias noise (reference binary.py:54-64)."""
        if self.seed is None:
            self.set_seed()
        if noise_scale is not None:
            self.set_noise_scale(noise_scale)
        self.weight_noise = booleanOperations.sample_bits(self.bernoulli_probabilities(), self.directions, self.dtype,
                                                          self.seed, self.uniforms)
        self.bias_noise = torch.empty((self.directions, self.out_degree), dtype=_F16, device=self.weight.device)
        C.call("nes_binarized_bias_noise", C.ptr(self.bias_noise), self.bias_noise.numel(),
               (int(self.seed) * 4 + 1) & (2 ** 64 - 1), self._member_groups(self.member_offset, self.out_degree, 4),
               C.stream())

    def update(self, weights, l1=0, l2=1e-3):
        """Centred fitness -> weighted bit sum (+ l1 / l2) into ``weight.grad`` and ``weights @ bias_noise`` into
        ``bias.grad``, all in one library call (reference binary.py:67-77)."""
        if weights.numel() != self.directions:
            raise RuntimeError("update weights must have one entry per direction")
        fitness = C.require_cuda(weights.detach().float(), "weights", torch.float32)
        bits = C.require_cuda(self.weight_noise, "weight_noise")
        rows, words = bits.shape[1], bits.shape[2]
        grad = torch.empty((rows, self.in_degree), dtype=_F16, device=bits.device)
        bias_grad = beta = None
        if self.bias is not None:
            beta = C.require_cuda(self.bias_noise, "bias_noise", _F16)
            bias_grad = torch.empty(self.out_degree, dtype=_F16, device=bits.device)
        wb = _word_bits(bits.dtype)
        nbytes = C.call("nes_binarized_update_scratch_bytes", self.directions, rows, words, wb)
        buf = C.scratch(nbytes, bits.device)
        C.call("nes_binarized_update", C.ptr(bits), C.ptr(fitness), _half_ptr(self.weight, "weight"), C.ptr(beta),
               C.ptr(grad), C.ptr(bias_grad), self.directions, rows, words, self.in_degree, self.out_degree, wb,
               float(l1), float(l2), C.ptr(buf), nbytes, C.stream())
        self.weight.grad = grad
        if self.bias is not None:
            self.bias.grad = bias_grad

    def _out_kind(self):
        """0 = integer activation, 1 = bool bits, 2 = packed bits."""
        if not self.threshold:
            return 0
        return 2 if self.packed_output else 1


class BinarizedLinear(Binarized):
    """activation = 2 * popcount(W_d ^ x_d) - in_features, optionally compared with
    bias + bias_noise (+ batch mean) (reference binary.py:80-108)."""

    def __init__(self, in_features, out_features, directions, threshold=True, batch_norm=False,
                 dtype=torch.int64, device="cuda"):
        Binarized.__init__(self, in_features, out_features, directions, threshold, dtype, device)
        self.in_features = in_features
        self.out_features = out_features
        self.weight = Parameter(torch.zeros(out_features, in_features, dtype=_F16, device=device))
        if threshold:
            self.bias = Parameter(torch.zeros(out_features, dtype=_F16, device=device))
        self.batch_norm = batch_norm
        self.reset_parameters()

    def forward(self, input):
        if not self.perturbed_flag:
            raise NotImplementedError
        x = booleanOperations.pack(input, self.dtype) if input.dtype == torch.bool else C.require_cuda(input, "input")
        bits = C.require_cuda(self.weight_noise, "weight_noise")
        D, out_f, words = bits.shape
        wb = _word_bits(bits.dtype)
        if x.dtype != bits.dtype or x.numel() != D * words:
            raise RuntimeError("expected one packed input vector of %d %s words per member" % (words, bits.dtype))
        kind = self._out_kind()
        fused = words * (wb // 8) % 16 == 0 and words * (wb // 8) <= 512 and D <= 65535
        if not fused:
            return self._generic_forward(x, bits, kind)
        if kind == 0:
            out = torch.empty((D, out_f), dtype=torch.int32, device=bits.device)
        elif kind == 1:
            out = torch.empty((D, out_f), dtype=torch.bool, device=bits.device)
        else:
            out = torch.empty((D, (out_f + wb - 1) // wb), dtype=self.dtype, device=bits.device)
        norm = 1 if (self.batch_norm and kind) else 0
        nbytes = C.call("nes_binarized_linear_fwd_scratch_bytes", D, out_f, norm)
        buf = C.scratch(nbytes, bits.device)
        C.call("nes_binarized_linear_fwd", C.ptr(bits), C.ptr(x), _half_ptr(self.bias, "bias") if kind else None,
               C.ptr(C.require_cuda(self.bias_noise, "bias_noise", _F16)) if kind else None, C.ptr(out), D, out_f, words,
               self.in_features, wb, kind, norm, C.ptr(buf), nbytes, C.stream())
        return out

    def _generic_forward(self, x, bits, kind):
        """Row lengths the streaming kernel does not take: counts from the tiled product, then the shared epilogue
        (a linear layer is a convolution with one position per member ... with the batch mean taken over members)."""
        D, out_f, _ = bits.shape
        counts = booleanOperations.bmm(bits, x.view(D, -1, 1)).view(D, 1, out_f)
        if kind and self.batch_norm:
            raise NotImplementedError("batch_norm needs packed rows that are multiples of 16 bytes")
        return _threshold_counts(self, counts, self.in_features, False, kind).view(D, -1)


def _threshold_counts(layer, counts, offset, batch_norm, kind):
    """Launch the epilogue on counts (P, S, N): the activation 2 * counts - offset in place (kind 0), or its
    comparison with the layer's thresholds as bool (P, S, N) / packed (P, S, words)."""
    P, S, N = counts.shape
    wb = _word_bits(layer.dtype)
    if kind == 0:
        C.call("nes_binarized_conv_epilogue", C.ptr(counts), None, None, C.ptr(counts), P, S, N, int(offset), wb, 0, 0,
               None, C.stream())
        return counts
    if kind == 1:
        out = torch.empty((P, S, N), dtype=torch.bool, device=counts.device)
    else:
        out = torch.empty((P, S, (N + wb - 1) // wb), dtype=layer.dtype, device=counts.device)
    sums = torch.empty((P, N), dtype=torch.float32, device=counts.device) if batch_norm else None
    C.call("nes_binarized_conv_epilogue", C.ptr(counts), _half_ptr(layer.bias, "bias"),
           C.ptr(C.require_cuda(layer.bias_noise, "bias_noise", _F16)), C.ptr(out), P, S, N, int(offset), wb, kind,
           1 if batch_norm else 0, C.ptr(sums), C.stream())
    return out


class BinarizedConv2d(Binarized):
    """Packed NHWC convolution with per-member binary filters (reference binary.py:112-166)."""

    def __init__(self, in_channels, out_channels, directions, kernel_size, stride=1, padding=0, dilation=1,
                 groups=1, threshold=True, batch_norm=True, padding_mode='zeros', dtype=torch.int64, device="cuda"):
        Binarized.__init__(self, in_channels, out_channels, directions, threshold, dtype, device)
        if dilation != 1 or groups != 1 or padding_mode != "zeros":
            raise NotImplementedError
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.stride = stride
        self.padding = padding
        self.kernel_size = (kernel_size, kernel_size) if isinstance(kernel_size, int) else kernel_size
        taps = self.kernel_size[0] * self.kernel_size[1]
        self.weight = Parameter(torch.zeros(out_channels * taps, in_channels, dtype=_F16, device=device))
        if threshold:
            self.bias = Parameter(torch.zeros(out_channels, dtype=_F16, device=device))
        self.batch_norm = batch_norm
        self.weight_noise_reshaped = None
        self.reset_parameters()

    def set_noise(self, noise_scale=None):
        Binarized.set_noise(self, noise_scale)
        # (D, out*kx*ky, Cw) -> (D, kx*ky*Cw, out): the filter layout conv() expects (reference binary.py:136-137)
        D, kx, ky = self.directions, *self.kernel_size
        self.weight_noise_reshaped = (self.weight_noise.view(D, self.out_channels, kx, ky, -1)
                                      .permute(0, 2, 3, 4, 1).reshape(D, -1, self.out_channels).contiguous())

    def forward(self, input):
        if not self.perturbed_flag:
            raise NotImplementedError
        if input.dtype == torch.bool:
            x = booleanOperations.pack(input.reshape(-1, self.in_channels), self.dtype).view(*input.shape[:3], -1)
        else:
            x = input
        taps_bits = self.in_channels * self.kernel_size[0] * self.kernel_size[1]
        geom = (*self.kernel_size, self.padding, self.padding, self.stride, self.stride)
        kind = self._out_kind()
        if kind and not self.batch_norm:
            # the reference's integer-threshold path (binary.py:156-157): 2 * conv > int(bias + bias_noise) + offset
            thresh = torch.empty((self.directions, self.out_channels), dtype=torch.int32, device=x.device)
            C.call("nes_binarized_int_threshold", _half_ptr(self.bias, "bias"),
                   C.ptr(C.require_cuda(self.bias_noise, "bias_noise", _F16)), C.ptr(thresh), self.directions,
                   self.out_channels, taps_bits, C.stream())
            bools = booleanOperations.conv_act(x, self.weight_noise_reshaped, thresh, *geom)
            if kind == 1:
                return bools
            return booleanOperations.pack(bools.view(-1, self.out_channels), self.dtype).view(*bools.shape[:3], -1)
        counts = booleanOperations.conv(x, self.weight_noise_reshaped, *geom)
        P, h, w, N = counts.shape
        out = _threshold_counts(self, counts.view(P, h * w, N), taps_bits, self.batch_norm, kind)
        return out.view(P, h, w, -1)

    def free_memory(self):
        Perturbed.free_memory(self)
        self.weight_noise_reshaped = None


class BinarizedMaxPool2d(nn.Module):
    """OR-pooling of packed NHWC bits (reference binary.py:168-182)."""

    def __init__(self, kernel_size=(2, 2), padding=(0, 0), stride=(2, 2), dtype=torch.int64):
        nn.Module.__init__(self)
        self.kernel_size = kernel_size
        self.padding = padding
        self.stride = stride
        self.dtype = dtype

    def forward(self, input):
        x = input
        if x.dtype == torch.bool:
            x = booleanOperations.pack(x.reshape(-1, x.size(3)), self.dtype).view(*x.shape[:3], -1)
        return booleanOperations.max_pool2d(x, *self.kernel_size, *self.padding, *self.stride)
