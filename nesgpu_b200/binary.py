"""Bit-packed population layers: host-side mirror of the reference's ``modules/binary.py``
(NESgpu) over :mod:`nesgpu_b200.boolean_operations`.

Each member owns a weight matrix of +-1 values drawn as Bernoulli(sigmoid(5 W / mean|W|)) and
stored as packed bits ``(directions, out, ceil(in/bits))``; activations are bools / packed
bits; the product is an XOR-popcount.  Only population mode exists (as in the reference,
``forward`` with the perturbed flag off raises).
"""
import torch
from torch import nn
from torch.nn.parameter import Parameter

from . import boolean_operations as booleanOperations
from .base import Perturbed, PerturbedModel  # noqa: F401  (re-exported like the reference's star import)


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


class Binarized(nn.Module, Perturbed):
    """State shared by the binary layers (reference binary.py:32-77)."""

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

    def reset_parameters(self):
        with torch.no_grad():
            self.weight.fill_(0)
            if self.threshold:
                self.bias.fill_(0)

    def bernoulli_probabilities(self):
        """sigmoid(5 W / (mean|W| + 1e-5)) as fp16 (reference binary.py:59-60)."""
        norm_weight = self.weight.detach() / (self.weight.detach().abs().mean() + 1e-5) * 5
        return torch.sigmoid(norm_weight.float()).half()

    def set_noise(self, noise_scale=None):
        if self.seed is None:
            self.set_seed()
        if noise_scale is not None:
            self.set_noise_scale(noise_scale)
        P = self.bernoulli_probabilities()
        self.weight_noise = booleanOperations.sample_bits(P, self.directions, self.dtype, self.seed, self.uniforms)
        self.bias_noise = (torch.rand(size=(self.directions, self.out_degree), dtype=torch.float16,
                                      device=self.weight.device) - .5) * 6

    def update(self, weights, l1=0, l2=1e-3):
        """Reference binary.py:67-77: centre the fitness, weighted bit sum, l1/l2, bias gradient."""
        weights = weights.type(torch.float16)
        weights = (weights - weights.mean())
        self.weight.grad = booleanOperations.weighted_sum(self.weight_noise, weights, self.in_degree)
        if l1:
            self.weight.grad += l1 * torch.sign(self.weight.detach())
        if l2:
            self.weight.grad += l2 * self.weight.detach()
        if self.bias is not None:
            self.bias.grad = weights @ self.bias_noise


class BinarizedLinear(Binarized):
    """activation = 2 * popcount(W_d ^ x_d) - in_features, optionally compared with
    bias + bias_noise (+ batch mean) (reference binary.py:80-108)."""

    def __init__(self, in_features, out_features, directions, threshold=True, batch_norm=False,
                 dtype=torch.int64, device="cuda"):
        Binarized.__init__(self, in_features, out_features, directions, threshold, dtype, device)
        self.in_features = in_features
        self.out_features = out_features
        self.weight = Parameter(torch.zeros(out_features, in_features, dtype=torch.float16, device=device))
        if threshold:
            self.bias = Parameter(torch.zeros(out_features, dtype=torch.float16, device=device))
        self.batch_norm = batch_norm
        self.reset_parameters()

    def forward(self, input):
        if not self.perturbed_flag:
            raise NotImplementedError
        packed_input = booleanOperations.pack(input, self.dtype) if input.dtype == torch.bool else input
        counts = booleanOperations.bmm(self.weight_noise, packed_input.view(self.directions, -1, 1)).squeeze(dim=2)
        activation = 2 * counts - self.in_features
        if self.threshold:
            thresh = (self.bias + self.bias_noise)
            if self.batch_norm:
                thresh = thresh + activation.type(torch.float16).mean(dim=0, keepdim=True)
            return activation > thresh
        return activation


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
        self.weight = Parameter(torch.zeros(out_channels * self.kernel_size[0] * self.kernel_size[1], in_channels,
                                            dtype=torch.float16, device=device))
        if threshold:
            self.bias = Parameter(torch.zeros(out_channels, dtype=torch.float16, device=device))
        self.batch_norm = batch_norm
        self.weight_noise_reshaped = None
        self.reset_parameters()

    def set_noise(self, noise_scale=None):
        Binarized.set_noise(self, noise_scale)
        # (D, out*kx*ky, Cw) -> (D, kx*ky*Cw, out): the filter layout conv() expects (binary.py:136-137)
        w = self.weight_noise.view(self.directions, self.out_channels, *self.kernel_size, -1)
        self.weight_noise_reshaped = w.permute([0, 2, 3, 4, 1]).reshape(self.directions, -1, self.out_channels).contiguous()

    def forward(self, input):
        if not self.perturbed_flag:
            raise NotImplementedError
        if input.dtype == torch.bool:
            packed_input = booleanOperations.pack(input.reshape(-1, self.in_channels), self.dtype).view(*input.shape[:3], -1)
        else:
            packed_input = input
        offset = self.in_channels * self.kernel_size[0] * self.kernel_size[1]
        geom = (*self.kernel_size, self.padding, self.padding, self.stride, self.stride)
        if self.threshold:
            if self.batch_norm:
                activation = 2 * booleanOperations.conv(packed_input, self.weight_noise_reshaped, *geom) - offset
                thresh = self.bias + self.bias_noise + activation.type(torch.float16).mean(dim=[1, 2])
                return activation > thresh.unsqueeze(1).unsqueeze(1)
            return booleanOperations.conv_act(packed_input, self.weight_noise_reshaped,
                                              (self.bias + self.bias_noise).type(torch.int32) + offset, *geom)
        return 2 * booleanOperations.conv(packed_input, self.weight_noise_reshaped, *geom) - offset

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
        if input.dtype == torch.bool:
            packed_input = booleanOperations.pack(input.reshape(-1, input.size(3)), self.dtype).view(*input.shape[:3], -1)
        else:
            packed_input = input
        return booleanOperations.max_pool2d(packed_input, *self.kernel_size, *self.padding, *self.stride)
