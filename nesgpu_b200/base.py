"""Population-batched perturbed layers on B200 kernels.

Host-side mirror of the reference's ``modules/base.py`` (NESgpu): the same class names,
constructor signatures, public attributes (``weight_noise``, ``bias_noise``,
``input_permutations``, ``output_permutations``, ``perturbed_flag`` ...) and methods
(``set_noise``, ``forward``, ``update`` ...), so user code written for the reference runs
unchanged.  All arithmetic happens in the CUDA library behind ``include/nesgpu_b200.h``;
this file only keeps state, validates shapes and launches.  Tensors must live on a CUDA
device and be fp32 -- there is no CPU path.

Batch layout (reference ``modules/base.py:357,368,490``): row ``b = r * directions + d``.
"""
import random

import torch
import torch.nn.functional as F
from torch import nn
from torch.nn.modules.utils import _pair

from . import _cabi as C

_F32 = torch.float32


def _opt(t):
    return None if t is None else C.require_cuda(t.detach(), "parameter", _F32)


def _grad_destination(param):
    """Where an update may write ``param``'s gradient instead of a fresh tensor: the slice of an all-reduce bucket
    that :mod:`nesgpu_b200.dist` attached to the parameter.  Only while ``.grad`` is empty (an accumulating update
    must not overwrite what ``.grad`` already holds, which may be that very slice)."""
    view = getattr(param, "_nes_grad_out", None)
    if view is None or param.grad is not None:
        return None
    if view.shape != param.shape or view.device != param.device or view.dtype != _F32 or not view.is_contiguous():
        return None
    return view


class PerturbedModel:
    """Wraps a model whose layers derive from :class:`Perturbed` (reference ``base.py:9-41``).

    ``forward`` runs the model with every perturbed layer switched to population mode; a
    method name that :class:`Perturbed` defines is broadcast to all perturbed layers; any
    other attribute is looked up on the model and called in population mode."""

    def __init__(self, model, directions):
        self.model = model
        self.directions = directions
        self.perturbed_layers = [m for m in model.modules() if isinstance(m, Perturbed)]

    def _population_mode(self, on):
        for layer in self.perturbed_layers:
            layer.perturbed_flag = on

    def forward(self, input, *args):
        self._population_mode(True)
        try:
            return self.model.forward(input, *args)
        finally:
            self._population_mode(False)

    def __getattr__(self, name):
        if hasattr(Perturbed, name):
            def broadcast(*args, **kwargs):
                for layer in self.perturbed_layers:
                    getattr(layer, name)(*args, **kwargs)
            return broadcast

        def in_population_mode(*args, **kwargs):
            self._population_mode(True)
            try:
                return getattr(self.model, name)(*args, **kwargs)
            finally:
                self._population_mode(False)
        return in_population_mode


class Perturbed:
    """Dense per-member Gaussian noise (reference ``base.py:44-138``).

    ``weight_noise`` is ``(directions, *weight.shape)``, ``bias_noise`` ``(directions, *bias.shape)``,
    both already scaled by ``noise_scale``.  ``options["direct"]`` stores ``weight + noise``
    instead (reference ``base.py:67-81``)."""

    def __init__(self, directions, antithetic=False, options={}):
        self.directions = directions
        self.perturbed_flag = False
        self.noise_scale = None
        self.seed = None
        self.antithetic = antithetic
        self.options = options
        self.member_offset = 0
        self.free_memory()

    # -- state ---------------------------------------------------------------------------
    def set_noise_scale(self, noise_scale):
        self.noise_scale = noise_scale

    def set_member_offset(self, first_member=0):
        """Global index of this layer's member 0 when the population is sharded over processes.

        Per-member draws (dense noise, bias noise, permutations, sign flips) are keyed on
        ``member_offset + d``, so ranks that share a seed draw disjoint members -- with row lengths that are
        multiples of the generator's group size, exactly the slice a single process would draw -- while the
        noise every member shares (``Permuted`` / ``Synthetic`` ``weight_noise``) stays identical on all ranks."""
        self.member_offset = int(first_member)

    def set_seed(self, seed=None):
        self.seed = random.randrange(100000000) if seed is None else seed

    def allocate_weight(self):
        self.weight_noise = torch.empty((self.directions,) + tuple(self.weight.shape),
                                        device=self.weight.device, dtype=self.weight.dtype)

    def allocate_bias(self):
        if self.bias is not None:
            self.bias_noise = torch.empty((self.directions,) + tuple(self.bias.shape),
                                          device=self.bias.device, dtype=self.bias.dtype)

    def allocate_memory(self):
        self.allocate_weight()
        self.allocate_bias()

    def free_memory(self):
        self.weight_noise = None
        if getattr(self, "bias", None) is not None:
            self.bias_noise = None

    def _prepare_noise(self, noise_scale):
        if self.seed is None:
            self.set_seed()
        if noise_scale is not None:
            self.set_noise_scale(noise_scale)
        if self.weight_noise is None:
            self.allocate_memory()

    @staticmethod
    def _member_groups(first_member, per_member, group):
        """Counter offset (in generator groups of ``group`` values) of member ``first_member`` in a
        ``(members, per_member)`` tensor: the exact position when rows are whole groups, otherwise a
        spacing that keeps the ranges of different ranks apart."""
        if not first_member:
            return 0
        if per_member % group == 0:
            return first_member * (per_member // group)
        return first_member * (per_member // group + 2)

    @classmethod
    def _fill_normal(cls, t, std, seed, stream_id, first_member=0):
        """N(0, std^2) from the device generator; ``stream_id`` separates the tensors of a layer,
        ``first_member`` shifts a per-member tensor to its place in the whole population."""
        C.require_cuda(t, "noise tensor", _F32)
        per_member = t[0].numel() if t.dim() and t.shape[0] else 1
        C.call("nes_fill_normal", C.ptr(t), t.numel(), 0.0, float(std), int(seed) & (2 ** 64 - 1),
               (int(stream_id) << 40) + cls._member_groups(first_member, per_member, 4), C.stream())

    def set_noise(self, noise_scale=None):
        """Draw fresh noise on the device (reference ``base.py:59-85``)."""
        self._prepare_noise(noise_scale)
        direct = bool(self.options.get("direct"))
        pairs = [(self.weight_noise, self.weight, 0)]
        if self.bias is not None:
            pairs.append((self.bias_noise, self.bias, 1))
        for noise, param, sid in pairs:
            if direct and self.antithetic:
                half = self.directions // 2
                self._fill_normal(noise[:half], self.noise_scale, self.seed, sid, self.member_offset)
                noise[half:] = -noise[:half]
            else:
                self._fill_normal(noise, self.noise_scale, self.seed, sid, self.member_offset)
            if direct:
                noise += param.detach()

    # -- update --------------------------------------------------------------------------
    def _direct_param(self, param):
        """With "direct" storage the tensors hold ``param + noise`` (reference ``base.py:111-117``); the
        reduction kernel then subtracts the parameter from every member's row as it streams it."""
        if not self.options.get("direct"):
            return None
        if self.antithetic:
            raise NotImplementedError("direct + antithetic update is inconsistent in the reference "
                                      "(modules/base.py:113-118) and is not provided")
        return param.detach()

    @staticmethod
    def _weighted_sum(noise, weights, param, l1, l2, direct_param=None, out=None):
        """sum_d weights[d] * noise[d] (+ l1 sign(param) + l2 param) as a tensor shaped like noise[0] (written
        into ``out`` when given)."""
        noise = C.require_cuda(noise, "noise", _F32)
        weights = C.require_cuda(weights, "weights", _F32)
        D = noise.shape[0]
        n = noise[0].numel() if D else 0
        if weights.numel() != D:
            raise RuntimeError("update weights must have one entry per direction")
        if out is None:
            out = torch.empty(noise.shape[1:], device=noise.device, dtype=_F32)
        nbytes = C.call("nes_perturbed_update_scratch_bytes", D, n)
        buf = C.scratch(nbytes, noise.device)
        reg = C.ptr(_opt(param)) if (l1 or l2) else None
        if direct_param is not None:
            C.call("nes_perturbed_update_direct", C.ptr(noise), C.ptr(weights),
                   C.ptr(C.require_cuda(direct_param, "parameter", _F32)), reg, C.ptr(out), D, n, float(l1), float(l2),
                   C.ptr(buf), nbytes, C.stream())
        else:
            C.call("nes_perturbed_update", C.ptr(noise), C.ptr(weights), reg, C.ptr(out), D, n, float(l1), float(l2),
                   C.ptr(buf), nbytes, C.stream())
        return out

    def weight_grad(self, weights):
        return self._weighted_sum(self.weight_noise, weights, None, 0, 0, self._direct_param(self.weight))

    def weight_grad_columns(self, weights, lo, hi, out, l1=0, l2=0):
        """Entries [lo, hi) of the flattened weight gradient, written into ``out`` (a contiguous fp32 tensor of
        hi - lo elements): the block-by-block form of :meth:`weight_grad` for dense per-member noise, so that a
        finished block can go to an all-reduce while the next one streams."""
        if self.options.get("direct"):
            raise NotImplementedError("column blocks are not provided for direct storage")
        noise = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        weights = C.require_cuda(weights, "weights", _F32)
        D = noise.shape[0]
        n = noise[0].numel()
        if not (0 <= lo <= hi <= n) or out.numel() != hi - lo or not out.is_contiguous():
            raise RuntimeError("bad column block")
        nbytes = C.call("nes_perturbed_update_scratch_bytes", D, hi - lo)
        buf = C.scratch(nbytes, noise.device)
        reg = _opt(self.weight).view(-1)[lo:hi] if (l1 or l2) else None
        C.call("nes_perturbed_update_columns", noise.data_ptr() + 4 * lo, C.ptr(weights), C.ptr(reg), C.ptr(out),
               D, hi - lo, n, float(l1), float(l2), C.ptr(buf), nbytes, C.stream())
        return out

    def _weight_grad_regularised(self, weights, l1, l2, out=None):
        return self._weighted_sum(self.weight_noise, weights, self.weight, l1, l2, self._direct_param(self.weight), out)

    def update(self, weights, l1=0, l2=0):
        """Accumulate the fitness-weighted noise sum into ``.grad`` (reference ``base.py:120-138``)."""
        grad = self._weight_grad_regularised(weights, l1, l2, _grad_destination(self.weight))
        self.weight.grad = grad if self.weight.grad is None else self.weight.grad + grad
        if self.bias is None:
            return grad
        bias_grad = self._weighted_sum(self.bias_noise, weights, None, 0, 0, self._direct_param(self.bias),
                                       _grad_destination(self.bias))
        self.bias.grad = bias_grad if self.bias.grad is None else self.bias.grad + bias_grad
        return grad, bias_grad

    # -- helpers shared by the layer classes ------------------------------------------------
    def _repeats(self, batch):
        if batch % self.directions:
            raise RuntimeError("batch size %d is not a multiple of directions %d" % (batch, self.directions))
        return batch // self.directions


def _resolve_permutation(in_degree, out_degree, permutation, in_sparsity, out_sparsity):
    """Which sides are permuted and how many noise rows/columns exist (reference ``base.py:148-184``)."""
    if permutation == "auto":
        if in_sparsity:
            permutation = "both" if out_sparsity else "in"
        elif out_sparsity:
            permutation = "out"
        elif 1 < in_degree < 32 and 1 < out_degree < 32:
            permutation = "both"
        else:
            permutation = "in" if in_degree > out_degree else "out"
    if permutation not in ("in", "out", "both"):
        raise NotImplementedError("Permutation setting not recognized")
    sides = {"in": permutation != "out", "out": permutation != "in"}
    kept = {}
    for side, degree, sp in (("in", in_degree, in_sparsity), ("out", out_degree, out_sparsity)):
        if isinstance(sp, float):
            sp = max(1, int(sp * degree))
        if sp:
            sides[side] = True
        kept[side] = sp if sp else degree
    return sides["in"], sides["out"], kept["in"], kept["out"]


class Permuted(Perturbed):
    """One shared noise tensor ``(out_sparsity, in_sparsity, ...)`` re-used by every member
    through per-member int16 permutations of the inputs and/or outputs (reference
    ``base.py:142-267``)."""

    def __init__(self, in_degree, out_degree, directions, antithetic=False, options={},
                 permutation="auto", in_sparsity=0, out_sparsity=0):
        Perturbed.__init__(self, directions, antithetic, options)
        (self.permute_inputs, self.permute_outputs,
         self.in_sparsity, self.out_sparsity) = _resolve_permutation(in_degree, out_degree, permutation,
                                                                     in_sparsity, out_sparsity)
        self.in_degree = in_degree
        self.out_degree = out_degree
        if max(in_degree, out_degree) > 32767:
            raise NotImplementedError("permutation tables are int16: degrees above 32767 are not supported")
        if options.get("combined") and self.permute_inputs and self.permute_outputs:
            raise NotImplementedError("Can't do combined multiplication with both input and output permutations")

    def allocate_weight(self):
        self.weight_noise = torch.empty((self.out_sparsity, self.in_sparsity) + tuple(self.weight.shape[2:]),
                                        device=self.weight.device, dtype=self.weight.dtype)

    def free_memory(self):
        Perturbed.free_memory(self)
        self.input_permutations = None
        self.output_permutations = None

    def _sample_permutations(self, n, keep, stream_id):
        out = torch.empty((self.directions, keep), dtype=torch.int16, device=self.weight.device)
        C.call("nes_sample_permutations", C.ptr(out), self.directions, n, keep,
               1 if self.options.get("allow_repeats") else 0,
               (int(self.seed) * 4 + stream_id) & (2 ** 64 - 1), self.member_offset, C.stream())
        return out

    def set_noise(self, noise_scale=None):
        """Shared noise, bias noise and permutations, all drawn on the device (reference
        ``base.py:197-227``, which loops ``torch.randperm`` on the CPU once per member)."""
        self._prepare_noise(noise_scale)
        rescale = (self.out_degree * self.in_degree / self.out_sparsity / self.in_sparsity) ** .5
        self._fill_normal(self.weight_noise, self.noise_scale * rescale, self.seed, 0)
        if self.bias is not None:
            self._fill_normal(self.bias_noise, self.noise_scale, self.seed, 1, self.member_offset)
        if self.permute_outputs:
            self.output_permutations = self._sample_permutations(self.out_degree, self.out_degree, 2)
        if self.permute_inputs:
            self.input_permutations = self._sample_permutations(self.in_degree, self.in_sparsity, 3)

    # index_select helpers kept for API parity (reference base.py:229-240); not on the fused path
    def _flat_index(self, perms, degree, device):
        return (perms.long() + (torch.arange(self.directions, device=device) * degree).unsqueeze(1)).flatten()

    def apply_input_permutation(self, input):
        if not self.permute_inputs:
            return input
        return torch.index_select(input, 1, self._flat_index(self.input_permutations, self.in_degree, input.device))

    def apply_output_permutation(self, output):
        if not self.permute_outputs:
            return output
        return torch.index_select(output, 1, self._flat_index(self.output_permutations, self.out_degree, output.device))

    def _perms(self):
        pin = C.require_cuda(self.input_permutations, "input_permutations", torch.int16) if self.permute_inputs else None
        pout = C.require_cuda(self.output_permutations, "output_permutations", torch.int16) if self.permute_outputs else None
        return pin, pout

    def _permuted_update(self, weights, l1, l2, want_perm_weights=False, out=None):
        eps = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        weights = C.require_cuda(weights, "weights", _F32)
        if weights.numel() != self.directions:
            raise RuntimeError("update weights must have one entry per direction")
        pin, pout = self._perms()
        ksize = 1
        for s in self.weight.shape[2:]:
            ksize *= s
        grad = out if out is not None else torch.empty_like(self.weight, memory_format=torch.contiguous_format)
        pw = None
        if want_perm_weights:
            shape = (self.in_sparsity, self.in_degree) if pin is not None else (self.out_degree, self.out_sparsity)
            pw = torch.empty(shape, device=eps.device, dtype=_F32)
        nbytes = C.call("nes_permuted_update_scratch_bytes", self.in_degree, self.out_degree,
                        self.in_sparsity, self.out_sparsity)
        buf = C.scratch(nbytes, eps.device)
        C.call("nes_permuted_update", C.ptr(eps), C.ptr(weights), C.ptr(pin), C.ptr(pout),
               C.ptr(_opt(self.weight)) if (l1 or l2) else None, C.ptr(grad), C.ptr(pw),
               self.directions, self.in_degree, self.out_degree, self.in_sparsity, self.out_sparsity, ksize,
               float(l1), float(l2), C.ptr(buf), nbytes, C.stream())
        return grad, pw

    def update(self, weights, l1=0, l2=0):
        """Layers with output permutations only get weight gradient, l1 / l2 terms and bias gradient from one
        launch; everything else takes the generic route (reference ``base.py:120-138``)."""
        if self.permute_inputs or not self.permute_outputs or self.out_sparsity * 32 + 65536 > 200 * 1024:
            return Perturbed.update(self, weights, l1, l2)
        eps = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        weights = C.require_cuda(weights, "weights", _F32)
        if weights.numel() != self.directions:
            raise RuntimeError("update weights must have one entry per direction")
        _, pout = self._perms()
        ksize = 1
        for s in self.weight.shape[2:]:
            ksize *= s
        grad = _grad_destination(self.weight)
        if grad is None:
            grad = torch.empty_like(self.weight, memory_format=torch.contiguous_format)
        beta = bias_grad = None
        if self.bias is not None:
            beta = C.require_cuda(self.bias_noise, "bias_noise", _F32)
            bias_grad = _grad_destination(self.bias)
            if bias_grad is None:
                bias_grad = torch.empty_like(self.bias)
        C.call("nes_permuted_update_out", C.ptr(eps), C.ptr(weights), C.ptr(pout),
               C.ptr(_opt(self.weight)) if (l1 or l2) else None, C.ptr(beta), C.ptr(grad), C.ptr(bias_grad),
               self.directions, self.in_degree, self.out_degree, self.out_sparsity, ksize, float(l1), float(l2),
               C.stream())
        self.weight.grad = grad if self.weight.grad is None else self.weight.grad + grad
        if self.bias is None:
            return grad
        self.bias.grad = bias_grad if self.bias.grad is None else self.bias.grad + bias_grad
        return grad, bias_grad

    def get_permutation_weights(self, weights):
        """The scatter-add matrix of reference ``base.py:254-267`` for the single-sided modes."""
        if self.permute_inputs and self.permute_outputs:
            raise NotImplementedError("two-sided permutation weights are O((out*in)^2) in the reference "
                                      "(modules/base.py:243-253); weight_grad computes the gradient directly")
        return self._permuted_update(weights, 0, 0, want_perm_weights=True)[1]

    def weight_grad(self, weights):
        return self._permuted_update(weights, 0, 0)[0]

    def _weight_grad_regularised(self, weights, l1, l2, out=None):
        return self._permuted_update(weights, l1, l2, out=out)[0]


_TC_MODES = {"3xtf32": 3, "tf32": 1}


class _LinearMixin:
    def _tensor_core_base(self, x, y):
        """y = x W^T + b on the tensor cores when the layer's ``options["tc"]`` allows it.

        ``"3xtf32"`` (default; error-compensated, fp32-level accuracy), ``"tf32"`` (plain TF32,
        relative error ~1e-3: a stated reduced-precision mode) or ``"fp32"`` (CUDA cores).
        Returns False when the CUDA-core kernel has to be used (mode "fp32" or a row length that is
        not a multiple of 4, which the TMA descriptors cannot express)."""
        mode = self.options.get("tc", "3xtf32")
        if mode == "fp32" or self.in_features % 4 or x.shape[0] == 0:
            return False
        if mode not in _TC_MODES:
            raise NotImplementedError('options["tc"] must be "3xtf32", "tf32" or "fp32"')
        M, N, K = x.shape[0], self.out_features, self.in_features
        nbytes = C.call("nes_linear_fwd_tc_scratch_bytes", M, N, K, _TC_MODES[mode])
        buf = C.scratch(nbytes, x.device)
        C.call("nes_linear_fwd_tc", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)), C.ptr(y),
               M, N, K, _TC_MODES[mode], C.ptr(buf), nbytes, C.stream())
        return True

    def _flatten_rows(self, input):
        x = C.require_cuda(input, "input", _F32)
        if x.shape[-1] != self.in_features:
            raise RuntimeError("expected last dimension %d, got %d" % (self.in_features, x.shape[-1]))
        return x.reshape(-1, self.in_features), x.shape[:-1]

    def _plain_forward(self, input):
        x, lead = self._flatten_rows(input)
        y = torch.empty((x.shape[0], self.out_features), device=x.device, dtype=_F32)
        C.call("nes_linear_fwd", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)), C.ptr(y),
               x.shape[0], self.out_features, self.in_features, C.stream())
        return y.view(*lead, self.out_features)


class PerturbedLinear(nn.Linear, _LinearMixin, Perturbed):
    """``y = x W^T + b + s * (x E_d^T + beta_d)`` with one dense noise matrix per member
    (reference ``base.py:349-381``)."""

    def __init__(self, in_features, out_features, directions, bias=True, antithetic=False, options={}):
        nn.Linear.__init__(self, in_features, out_features, bias)
        Perturbed.__init__(self, directions, antithetic, options)

    def forward(self, input):
        if not self.perturbed_flag:
            return self._plain_forward(input)
        x, lead = self._flatten_rows(input)
        R = self._repeats(x.shape[0])
        direct = 1 if self.options.get("direct") else 0
        noise = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        beta = C.require_cuda(self.bias_noise, "bias_noise", _F32) if self.bias is not None else None
        y = torch.empty((x.shape[0], self.out_features), device=x.device, dtype=_F32)
        self.last_path = "fp32"
        if not direct and self._tensor_core_base(x, y):
            direct = 2          # y now holds x W^T + b; the streaming kernel adds the per-member term
            self.last_path = self.options.get("tc", "3xtf32")
        C.call("nes_perturbed_linear_fwd", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)),
               C.ptr(noise), C.ptr(beta), C.ptr(y), self.directions, R, self.in_features, self.out_features,
               1 if self.antithetic else 0, direct, C.stream())
        if direct == 1:
            return y.view(R, self.directions, self.out_features)
        return y.view(*lead, self.out_features)


class SparsePerturbedLinear(nn.Linear, _LinearMixin, Perturbed):
    """Sparse Gaussian noise: ``k`` non-zero noise entries per member and output row
    (reference ``README.md:12,29-30``; the reference snapshot ships no source for it).

    ``noise_indices`` is ``(directions, out, k)`` int32, ``weight_noise`` ``(directions, out, k)``
    with standard deviation ``noise_scale * sqrt(in / k)`` so that the per-row noise energy
    matches the dense layer.  Forward and update equal :class:`PerturbedLinear` on the
    densified noise."""

    def __init__(self, in_features, out_features, directions, bias=True, antithetic=False, options={}, k=1):
        nn.Linear.__init__(self, in_features, out_features, bias)
        self.k = k
        Perturbed.__init__(self, directions, antithetic, options)
        if options.get("direct"):
            raise NotImplementedError("direct storage is not defined for sparse noise")

    def allocate_weight(self):
        shape = (self.directions, self.out_features, self.k)
        self.weight_noise = torch.empty(shape, device=self.weight.device, dtype=self.weight.dtype)
        self.noise_indices = torch.empty(shape, device=self.weight.device, dtype=torch.int32)

    def free_memory(self):
        Perturbed.free_memory(self)
        self.noise_indices = None

    def set_noise(self, noise_scale=None):
        self._prepare_noise(noise_scale)
        self._fill_normal(self.weight_noise, self.noise_scale * (self.in_features / self.k) ** .5, self.seed, 0,
                          self.member_offset)
        if self.bias is not None:
            self._fill_normal(self.bias_noise, self.noise_scale, self.seed, 1, self.member_offset)
        u = torch.empty(self.noise_indices.shape, device=self.weight.device, dtype=_F32)
        C.call("nes_fill_uniform", C.ptr(u), u.numel(), 0.0, 1.0, (int(self.seed) * 4 + 2) & (2 ** 64 - 1),
               self._member_groups(self.member_offset, self.out_features * self.k, 4), C.stream())
        self.noise_indices = (u * self.in_features).clamp_(max=self.in_features - 1).to(torch.int32)

    def forward(self, input):
        if not self.perturbed_flag:
            return self._plain_forward(input)
        x, lead = self._flatten_rows(input)
        R = self._repeats(x.shape[0])
        val = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        idx = C.require_cuda(self.noise_indices, "noise_indices", torch.int32)
        beta = C.require_cuda(self.bias_noise, "bias_noise", _F32) if self.bias is not None else None
        y = torch.empty((x.shape[0], self.out_features), device=x.device, dtype=_F32)
        if self._tensor_core_base(x, y):
            # base product on the tensor cores (3xTF32 unless options["tc"] says otherwise), then the k-entry gather
            self.last_path = self.options.get("tc", "3xtf32")
            C.call("nes_sparse_noise_add", C.ptr(y), C.ptr(x), C.ptr(idx), C.ptr(val), C.ptr(beta), self.directions, R,
                   self.in_features, self.out_features, self.k, 1 if self.antithetic else 0, C.stream())
            return y.view(*lead, self.out_features)
        self.last_path = "fp32"
        C.call("nes_sparse_perturbed_linear_fwd", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)),
               C.ptr(idx), C.ptr(val), C.ptr(beta), C.ptr(y), self.directions, R, self.in_features,
               self.out_features, self.k, 1 if self.antithetic else 0, C.stream())
        return y.view(*lead, self.out_features)

    def _weight_grad_regularised(self, weights, l1, l2, out=None):
        val = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        idx = C.require_cuda(self.noise_indices, "noise_indices", torch.int32)
        weights = C.require_cuda(weights, "weights", _F32)
        grad = out if out is not None else torch.empty_like(self.weight)
        C.call("nes_sparse_perturbed_update", C.ptr(idx), C.ptr(val), C.ptr(weights),
               C.ptr(_opt(self.weight)) if (l1 or l2) else None, C.ptr(grad), self.directions,
               self.in_features, self.out_features, self.k, float(l1), float(l2), C.stream())
        return grad

    def weight_grad(self, weights):
        return self._weight_grad_regularised(weights, 0, 0)


class PermutedLinear(nn.Linear, _LinearMixin, Permuted):
    """``y = x W^T + b + s * (gather_out(gather_in(x) eps^T) + beta_d)`` (reference
    ``base.py:447-518``).  ``options["combined"]`` selects the same fused kernels: the
    reference's combined branches are algebraic re-arrangements of this sum (its combined
    input branch additionally drops ``beta`` and the antithetic sign, ``base.py:458-464``;
    that omission is not reproduced)."""

    def __init__(self, in_features, out_features, directions, bias=True, antithetic=False, options={},
                 permutation="auto", in_sparsity=0, out_sparsity=0):
        nn.Linear.__init__(self, in_features, out_features, bias)
        Permuted.__init__(self, in_features, out_features, directions, antithetic=antithetic, options=options,
                          permutation=permutation, in_sparsity=in_sparsity, out_sparsity=out_sparsity)

    # batch rows from which the one-product tensor-core form is chosen by default (64 row tiles of 128)
    SINGLE_PRODUCT_MIN_ROWS = 64 * 128

    def _single_product_mode(self, rows, pout):
        """Mode (1 = TF32, 2 = bf16, 3 = 3xTF32, 4 = split-bf16) of the one-product tensor-core forward, or 0 for the
        CUDA-core kernels.

        ``options["tc"]``: ``"bf16x3"`` / ``"3xtf32"`` / ``"tf32"`` / ``"bf16"`` force it, ``"fp32"`` forbids it; by
        default ("auto") the split-bf16 form (three products on bf16 hi / lo parts, fp32-level accuracy, half the
        operand bytes of 3xTF32) is taken for batches of at least ``SINGLE_PRODUCT_MIN_ROWS`` rows.  It needs a layer
        without output permutations."""
        mode = self.options.get("tc", "auto")
        if mode not in ("auto", "fp32", "bf16x3", "3xtf32", "tf32", "bf16"):
            raise NotImplementedError('options["tc"] must be "auto", "bf16x3", "3xtf32", "tf32", "bf16" or "fp32"')
        if mode == "fp32" or pout is not None or rows == 0:
            return 0
        if mode == "auto":
            return 4 if rows >= self.SINGLE_PRODUCT_MIN_ROWS else 0
        return {"bf16x3": 4, "3xtf32": 3, "tf32": 1, "bf16": 2}[mode]

    def _cluster_kernel_mode(self, x, R, pin):
        """Mode (3 = 3xTF32, 1 = TF32) of the one-launch tensor-core forward for layers without input
        permutations, or 0 when the CUDA-core kernels have to run (``options["tc"] = "fp32"``, or a shape the
        kernel does not cover).  ``"auto"`` and ``"3xtf32"`` give the error-compensated form that holds the fp32
        bar; ``"tf32"`` is the stated reduced-precision mode."""
        mode = self.options.get("tc", "auto")
        if pin is not None or mode in ("fp32", "bf16") or x.shape[0] == 0:
            return 0
        m = 1 if mode == "tf32" else 3
        if x.data_ptr() % 16 or self.weight.data_ptr() % 16 or self.weight_noise.data_ptr() % 16:
            return 0
        ok = C.call("nes_permuted_linear_out_fwd_tc_supported", self.directions, R, self.in_features,
                    self.out_features, self.out_sparsity, m)
        return m if ok else 0

    def forward(self, input):
        if not self.perturbed_flag:
            return self._plain_forward(input)
        x, lead = self._flatten_rows(input)
        R = self._repeats(x.shape[0])
        eps = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        beta = C.require_cuda(self.bias_noise, "bias_noise", _F32) if self.bias is not None else None
        pin, pout = self._perms()
        y = torch.empty((x.shape[0], self.out_features), device=x.device, dtype=_F32)
        mode = self._single_product_mode(x.shape[0], pout)
        cluster_mode = self._cluster_kernel_mode(x, R, pin)
        self.last_path = ("3xtf32" if cluster_mode == 3 else "tf32") if cluster_mode else (
            {1: "tf32", 2: "bf16", 3: "3xtf32", 4: "bf16x3"}[mode] if mode else "fp32")
        if cluster_mode:
            C.call("nes_permuted_linear_out_fwd_tc", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)),
                   C.ptr(eps), C.ptr(beta), C.ptr(pout), C.ptr(y), self.directions, R, self.in_features,
                   self.out_features, self.out_sparsity, 1 if self.antithetic else 0, cluster_mode, C.stream())
            return y.view(*lead, self.out_features)
        if mode:
            nbytes = C.call("nes_permuted_linear_fwd_tc_scratch_bytes", self.directions, R, self.in_features,
                            self.out_features, self.in_sparsity, mode)
            buf = C.scratch(nbytes, x.device)
            C.call("nes_permuted_linear_fwd_tc", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)),
                   C.ptr(eps), C.ptr(beta), C.ptr(pin), C.ptr(y), self.directions, R, self.in_features,
                   self.out_features, self.in_sparsity, self.out_sparsity, 1 if self.antithetic else 0, mode,
                   C.ptr(buf), nbytes, C.stream())
            return y.view(*lead, self.out_features)
        nbytes = C.call("nes_permuted_linear_fwd_scratch_bytes", self.directions, R, self.out_sparsity)
        buf = C.scratch(nbytes, x.device)
        C.call("nes_permuted_linear_fwd", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)), C.ptr(eps),
               C.ptr(beta), C.ptr(pin), C.ptr(pout), C.ptr(y), self.directions, R, self.in_features,
               self.out_features, self.in_sparsity, self.out_sparsity, 1 if self.antithetic else 0,
               C.ptr(buf), nbytes, C.stream())
        return y.view(*lead, self.out_features)


class _ConvMixin:
    def _geometry(self, x):
        if self.groups != 1:
            raise NotImplementedError("groups != 1 is not supported")
        if x.dim() != 4 or x.shape[1] != self.in_channels:
            raise RuntimeError("expected (B, %d, H, W) input, got %s" % (self.in_channels, tuple(x.shape)))
        if self.padding_mode != "zeros":
            x = F.pad(x, self._reversed_padding_repeated_twice, mode=self.padding_mode).contiguous()
            pad = (0, 0)
        else:
            pad = _pair(self.padding)
        kh, kw = self.kernel_size
        sh, sw = _pair(self.stride)
        dh, dw = _pair(self.dilation)
        H, W = x.shape[-2:]
        Ho = (H + 2 * pad[0] - dh * (kh - 1) - 1) // sh + 1
        Wo = (W + 2 * pad[1] - dw * (kw - 1) - 1) // sw + 1
        geom = (self.in_channels, H, W, self.out_channels, kh, kw, sh, sw, pad[0], pad[1], dh, dw)
        return x, geom, (Ho, Wo)

    def _plain_forward(self, input):
        x = C.require_cuda(input, "input", _F32)
        x, geom, (Ho, Wo) = self._geometry(x)
        y = torch.empty((x.shape[0], self.out_channels, Ho, Wo), device=x.device, dtype=_F32)
        C.call("nes_conv2d_fwd", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)), C.ptr(y),
               x.shape[0], *geom, C.stream())
        return y

    def _tensor_core_mode(self, geom=None, permuted=None):
        """``options["tc"]`` -> entry-point suffix of the tcgen05 path, or None for the CUDA-core kernel.

        ``"auto"`` (default) and ``"bf16x3"``: the split-bf16 three-product form, which holds the fp32 bar (relative
        error a few 1e-6), wherever the geometry is covered (stride 1, in_channels a multiple of 64, out_channels a
        multiple of 8 up to 128); ``"auto"`` falls back to exact fp32 on CUDA cores elsewhere.  ``"fp32"``: CUDA cores.
        ``"tf32"`` / ``"bf16"``: operands rounded to TF32 / bf16, fp32 accumulation -- stated reduced-precision modes
        with relative error ~1e-3 / ~3e-3."""
        mode = self.options.get("tc", "auto")
        if mode not in ("auto", "fp32", "tf32", "bf16", "bf16x3"):
            raise NotImplementedError('options["tc"] for convolutions must be "auto", "fp32", "bf16x3", "tf32" or "bf16"')
        if mode in ("auto", "bf16x3"):
            if geom is None:
                covered = False
            elif permuted is not None:          # (in_sparsity, out_sparsity, has input permutations)
                covered = C.call("nes_permuted_conv2d_fwd_bf16x3_supported", geom[0], geom[1], geom[2], geom[3], *geom[4:12],
                                 int(permuted[0]), int(permuted[1]), 1 if permuted[2] else 0) == 1
            else:
                covered = C.call("nes_conv2d_fwd_bf16x3_supported", geom[0], geom[1], geom[2], geom[3], *geom[4:12]) == 1
            if covered:
                return "bf16x3"
            if mode == "bf16x3":
                raise NotImplementedError('options["tc"] = "bf16x3" does not cover this geometry')
            return None
        return {"fp32": None, "tf32": "tc", "bf16": "bf16"}[mode]

    def _tc_scratch(self, x, R, geom, suffix):
        nbytes = C.call("nes_conv2d_fwd_%s_scratch_bytes" % suffix, self.directions, R, self.in_channels,
                        x.shape[-2], x.shape[-1], self.out_channels, self.kernel_size[0], self.kernel_size[1],
                        geom[8], geom[9])
        return C.scratch(nbytes, x.device), nbytes

    def _dense_forward(self, x, geom, out_hw, noise):
        R = self._repeats(x.shape[0])
        beta = C.require_cuda(self.bias_noise, "bias_noise", _F32) if self.bias is not None else None
        y = torch.empty((x.shape[0], self.out_channels) + out_hw, device=x.device, dtype=_F32)
        suffix = self._tensor_core_mode(geom)
        self.last_path = {None: "fp32", "tc": "tf32"}.get(suffix, suffix)
        if suffix and x.shape[0]:
            buf, nbytes = self._tc_scratch(x, R, geom, suffix)
            C.call("nes_perturbed_conv2d_fwd_" + suffix, C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)),
                   C.ptr(noise), C.ptr(beta), C.ptr(y), self.directions, R, *geom,
                   1 if self.antithetic else 0, C.ptr(buf), nbytes, C.stream())
            return y
        C.call("nes_perturbed_conv2d_fwd", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)),
               C.ptr(noise), C.ptr(beta), C.ptr(y), self.directions, R, *geom,
               1 if self.antithetic else 0, C.stream())
        return y


class PerturbedConv2d(nn.Conv2d, _ConvMixin, Perturbed):
    """Per member a convolution with ``weight + s * noise[d]`` (reference ``base.py:384-425``,
    which evaluates the noise term as one grouped convolution with ``groups * directions``
    groups)."""

    def __init__(self, in_channels, out_channels, kernel_size, directions, stride=1, padding=0, dilation=1,
                 groups=1, bias=True, antithetic=False, options={}, padding_mode='zeros'):
        nn.Conv2d.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups,
                           bias, padding_mode)
        Perturbed.__init__(self, directions, antithetic, options)
        if options.get("direct"):
            raise NotImplementedError("direct storage for PerturbedConv2d drops the bias noise in the reference "
                                      "(modules/base.py:401-409) and is not provided")

    def forward(self, input):
        if not self.perturbed_flag:
            return self._plain_forward(input)
        x = C.require_cuda(input, "input", _F32)
        x, geom, out_hw = self._geometry(x)
        return self._dense_forward(x, geom, out_hw, C.require_cuda(self.weight_noise, "weight_noise", _F32))


class PermutedConv2d(nn.Conv2d, _ConvMixin, Permuted):
    """Shared noise filter with per-member channel permutations (reference ``base.py:521-599``).
    Evaluated as one convolution per member with the effective filter
    ``W + s * eps[pi_out[d, k], pi_in^-1[d, c]]`` formed inside the kernel."""

    def __init__(self, in_channels, out_channels, kernel_size, directions, stride=1, padding=0, dilation=1,
                 groups=1, bias=True, antithetic=False, options={}, padding_mode='zeros', permutation="auto",
                 in_sparsity=0, out_sparsity=0):
        nn.Conv2d.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups,
                           bias, padding_mode)
        Permuted.__init__(self, in_channels, out_channels, directions, antithetic=antithetic, options=options,
                          permutation=permutation, in_sparsity=in_sparsity, out_sparsity=out_sparsity)

    def _dense_noise(self, eps, pin, pout):
        ksize = self.kernel_size[0] * self.kernel_size[1]
        E = torch.empty((self.directions, self.out_channels, self.in_channels) + tuple(self.kernel_size),
                        device=eps.device, dtype=_F32)
        C.call("nes_permuted_dense_noise", C.ptr(eps), C.ptr(pin), C.ptr(pout), C.ptr(E), self.directions,
               self.in_channels, self.out_channels, self.in_sparsity, self.out_sparsity, ksize, C.stream())
        return E

    def forward(self, input):
        """Two options beyond the reference's, both off by default:

        ``options["fuse"] = "relu_maxpool2"`` makes the layer return ``max_pool2d(relu(conv), 2)`` (the
        Conv -> ReLU -> MaxPool2d(2) block of the reference's models, ``models/mnistmodels.py:35-57``) so
        that the full-resolution activations never reach memory where a fused kernel exists;
        ``options["shared_input"] = True`` declares that every member sees the same images: the layer then
        takes ``(R, C, H, W)`` and returns the ``(R * directions, ...)`` population batch.  With both set and
        output permutations only, the two convolutions ``conv(x, W)`` and ``conv(x, eps)`` are computed once
        per image and the per-member work is a fused gather + add + ReLU + pool; the result is a
        channels-last tensor (``options["out_dtype"]`` = ``"tf32"`` rounds it to TF32, ``"bf16"`` stores bf16, for a
        tensor-core consumer; ``"bf16x2"`` stores bf16 with images 2q and 2q+1 interleaved by pixel, shape
        ``(R * directions / 2, 2 * C, H, W)``, which a following layer takes with ``options["in_layout"] =
        "bf16x2"`` to put two images into every tensor-core instruction)."""
        fuse = self.options.get("fuse")
        if fuse not in (None, "relu_maxpool2"):
            raise NotImplementedError('options["fuse"] must be "relu_maxpool2"')
        shared = bool(self.options.get("shared_input"))
        if not self.perturbed_flag:
            y = self._plain_forward(input)
            return F.max_pool2d(F.relu(y), 2) if fuse else y
        if shared:
            y = self._shared_fused_forward(input) if fuse else None
            if y is not None:
                return y
            input = input.unsqueeze(1).expand(input.shape[0], self.directions, *input.shape[1:]).reshape(
                input.shape[0] * self.directions, *input.shape[1:])
        y = self._fused_tc_forward(input) if fuse else None
        if y is not None:
            return y
        y = self._perturbed_forward(input)
        return F.max_pool2d(F.relu(y), 2) if fuse else y

    def _shared_fused_forward(self, input):
        """Shared images, output permutations only: one stacked convolution per image, then the fused
        per-member kernel.  Returns None when the case is not covered."""
        pin, pout = self._perms()
        if pin is not None or self.options.get("allow_repeats"):
            return None
        x = C.require_cuda(input, "input", _F32)
        x, geom, (Ho, Wo) = self._geometry(x)
        osp, cout = self.out_sparsity, self.out_channels
        if (cout + osp + 1) * (Ho * Wo + 1) * 4 + 80 * cout + 16 > 220 * 1024 or Ho < 2 or Wo < 2:
            return None
        eps = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        beta = C.require_cuda(self.bias_noise, "bias_noise", _F32) if self.bias is not None else None
        R, D = x.shape[0], self.directions
        stacked = torch.cat([self.weight.detach(), eps.view(osp, *self.weight.shape[1:])], dim=0).contiguous()
        z = torch.empty((R, cout + osp, Ho, Wo), device=x.device, dtype=_F32)
        C.call("nes_conv2d_fwd", C.ptr(x), C.ptr(stacked), None, C.ptr(z), R, geom[0], geom[1], geom[2], cout + osp,
               *geom[4:], C.stream())
        out = self.options.get("out_dtype", "fp32")
        if self.options.get("out_tf32"):
            out = "tf32"
        if out not in ("fp32", "tf32", "bf16", "bf16x2", "bf16x3"):
            raise NotImplementedError('options["out_dtype"] must be "fp32", "tf32", "bf16", "bf16x2" or "bf16x3"')
        if out == "bf16x2" and D % 2:
            raise NotImplementedError('options["out_dtype"] = "bf16x2" needs an even number of directions')
        lead = (2, R * D) if out == "bf16x3" else (R * D,)         # split form: a hi and a lo copy of the batch
        y = torch.empty(lead + (Ho // 2, Wo // 2, cout), device=x.device,
                        dtype=_F32 if out in ("fp32", "tf32") else torch.bfloat16)
        C.call("nes_shared_conv_pool_fwd", C.ptr(z), C.ptr(_opt(self.bias)), C.ptr(beta), C.ptr(pout), C.ptr(y),
               R, D, cout, osp, Ho, Wo, 1 if self.antithetic else 0,
               {"fp32": 0, "tf32": 1, "bf16": 2, "bf16x2": 3, "bf16x3": 4}[out], C.stream())
        if out == "bf16x3":
            return y.permute(0, 1, 4, 2, 3)                       # (2, B, C, H, W): bf16 hi and lo parts, channels-last
        if out == "bf16x2":
            # images 2q and 2q+1 interleaved by pixel: a channels-last tensor of R*D/2 "double" images
            return y.view(R * D // 2, Ho // 2, Wo // 2, 2 * cout).permute(0, 3, 1, 2)
        return y.permute(0, 3, 1, 2)

    def _fused_tc_forward(self, input):
        """Conv + ReLU + MaxPool2d(2) in one tensor-core kernel (``options["tc"]`` = ``"tf32"`` or ``"bf16"``, output permutations
        only, 32 input channels, stride 1 / no padding, one image per 128-column accumulator).  Takes the
        input channels-last without a copy.  Returns None when the case is not covered."""
        mode = self.options.get("tc")
        if self.options.get("in_layout") == "bf16x2":
            return self._fused_pair_forward(input)
        if mode not in ("tf32", "bf16", "bf16x3") or self.options.get("allow_repeats") or self.groups != 1:
            return None
        split = mode == "bf16x3"
        if split:
            # the split form takes the (2, B, C, H, W) bf16 hi / lo pair a shared-input layer stores with
            # out_dtype "bf16x3"; an ordinary fp32 batch is split here
            if isinstance(input, torch.Tensor) and input.dim() == 4 and input.dtype == _F32:
                hi = input.to(torch.bfloat16)
                input = torch.stack([hi, (input - hi.float()).to(torch.bfloat16)])
            if not (isinstance(input, torch.Tensor) and input.is_cuda and input.dim() == 5 and input.shape[0] == 2
                    and input.dtype == torch.bfloat16):
                return None
            pair, input = input, input[0]
        pin, pout = self._perms()
        kh, kw = self.kernel_size
        if (pin is not None or self.in_channels != 32 or self.out_channels > 64 or self.out_sparsity > 64
                or kh * kw > 9 or _pair(self.stride) != (1, 1) or _pair(self.dilation) != (1, 1)
                or self.padding_mode != "zeros" or _pair(self.padding) != (0, 0)):
            return None
        if not isinstance(input, torch.Tensor) or not input.is_cuda or input.dim() != 4:
            return None
        if input.dtype not in (_F32, torch.bfloat16):
            return None
        B, _, H, W = input.shape
        if H < kh or W < kw or B == 0:
            return None
        Hp, Wp = (H - kh + 1) // 2, (W - kw + 1) // 2
        if Hp < 1 or Wp < 1 or (2 * Hp - 1) * W + 2 * Wp > 128 or 128 + (kh - 1) * W + kw - 1 > 256:
            return None
        eps = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        beta = C.require_cuda(self.bias_noise, "bias_noise", _F32) if self.bias is not None else None
        R = self._repeats(B)
        if split:
            xs = pair.permute(0, 1, 3, 4, 2)
            if not xs.is_contiguous():
                xs = xs.contiguous()
            y = torch.empty((B, self.out_channels, Hp, Wp), device=xs.device, dtype=_F32)
            nbytes = C.call("nes_permuted_conv_pool_fwd_bf16x3_scratch_bytes", kh, kw)
            buf = C.scratch(nbytes, xs.device)
            self.last_path = "bf16x3"
            C.call("nes_permuted_conv_pool_fwd_bf16x3", C.ptr(xs[0]), C.ptr(xs[1]), C.ptr(_opt(self.weight)),
                   C.ptr(_opt(self.bias)), C.ptr(eps), C.ptr(beta), C.ptr(pout), C.ptr(y), self.directions, R, 32, H, W,
                   self.out_channels, kh, kw, self.out_sparsity, 1 if self.antithetic else 0, C.ptr(buf), nbytes,
                   C.stream())
            return y
        x = input.permute(0, 2, 3, 1)
        want = torch.bfloat16 if mode == "bf16" else _F32
        if x.dtype != want:
            x = x.to(want)
        if not x.is_contiguous():
            x = x.contiguous()
        y = torch.empty((B, self.out_channels, Hp, Wp), device=x.device, dtype=_F32)
        nbytes = C.call("nes_permuted_conv_pool_fwd_tc_scratch_bytes", kh, kw)
        buf = C.scratch(nbytes, x.device)
        self.last_path = mode
        C.call("nes_permuted_conv_pool_fwd_" + ("bf16" if mode == "bf16" else "tc"), C.ptr(x), C.ptr(_opt(self.weight)),
               C.ptr(_opt(self.bias)), C.ptr(eps),
               C.ptr(beta), C.ptr(pout), C.ptr(y), self.directions, R, 32, H, W, self.out_channels, kh, kw,
               self.out_sparsity, 1 if self.antithetic else 0, C.ptr(buf), nbytes, C.stream())
        return y

    def _fused_pair_forward(self, input):
        """The bf16 fused kernel with two images per tensor-core instruction: ``input`` is the ``"bf16x2"`` output of
        a shared-input layer, ``(B / 2, 64, 13, 13)`` bf16 channels-last.  No other form of this layer can read that
        layout, so an uncovered case is an error."""
        pin, pout = self._perms()
        ok = (self.options.get("tc") == "bf16" and pin is None and not self.options.get("allow_repeats")
              and self.groups == 1 and self.in_channels == 32 and self.out_channels <= 64 and self.out_sparsity <= 64
              and tuple(self.kernel_size) == (3, 3) and _pair(self.stride) == (1, 1) and _pair(self.dilation) == (1, 1)
              and self.padding_mode == "zeros" and _pair(self.padding) == (0, 0)
              and isinstance(input, torch.Tensor) and input.is_cuda and input.dtype == torch.bfloat16
              and input.dim() == 4 and tuple(input.shape[1:]) == (64, 13, 13))
        if not ok:
            raise NotImplementedError('options["in_layout"] = "bf16x2" needs options["tc"] = "bf16", output permutations '
                                      'only, 32 -> <= 64 channels, 3x3 filters and a (B/2, 64, 13, 13) bf16 input')
        x = input.permute(0, 2, 3, 1)
        if not x.is_contiguous():
            x = x.contiguous()
        B = 2 * input.shape[0]
        eps = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        beta = C.require_cuda(self.bias_noise, "bias_noise", _F32) if self.bias is not None else None
        R = self._repeats(B)
        y = torch.empty((B, self.out_channels, 5, 5), device=x.device, dtype=_F32)
        nbytes = C.call("nes_permuted_conv_pool_fwd_tc_scratch_bytes", 3, 3)
        buf = C.scratch(nbytes, x.device)
        C.call("nes_permuted_conv_pool_fwd_bf16x2", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)), C.ptr(eps),
               C.ptr(beta), C.ptr(pout), C.ptr(y), self.directions, R, 32, 13, 13, self.out_channels, 3, 3,
               self.out_sparsity, 1 if self.antithetic else 0, C.ptr(buf), nbytes, C.stream())
        return y

    def _perturbed_forward(self, input):
        x = C.require_cuda(input, "input", _F32)
        x, geom, out_hw = self._geometry(x)
        eps = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        pin, pout = self._perms()
        if pin is not None and self.options.get("allow_repeats"):
            # a repeated input channel makes the member's filter a sum of noise columns
            return self._dense_forward(x, geom, out_hw, self._dense_noise(eps, pin, pout))
        R = self._repeats(x.shape[0])
        beta = C.require_cuda(self.bias_noise, "bias_noise", _F32) if self.bias is not None else None
        y = torch.empty((x.shape[0], self.out_channels) + out_hw, device=x.device, dtype=_F32)
        suffix = self._tensor_core_mode(geom, (self.in_sparsity, self.out_sparsity, pin is not None))
        if suffix in ("bf16", "bf16x3") and pin is None and self.in_sparsity % 8:
            suffix = None if self.options.get("tc", "auto") == "auto" else suffix
        self.last_path = {None: "fp32", "tc": "tf32"}.get(suffix, suffix)
        if suffix and x.shape[0]:
            buf, nbytes = self._tc_scratch(x, R, geom, suffix)
            C.call("nes_permuted_conv2d_fwd_" + suffix, C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)),
                   C.ptr(eps), C.ptr(beta), C.ptr(pin), C.ptr(pout), C.ptr(y), self.directions, R, *geom,
                   self.in_sparsity, self.out_sparsity, 1 if self.antithetic else 0, C.ptr(buf), nbytes, C.stream())
            return y
        nbytes = C.call("nes_permuted_conv2d_fwd_scratch_bytes", self.directions, self.in_channels, self.out_channels)
        buf = C.scratch(nbytes, x.device)
        C.call("nes_permuted_conv2d_fwd", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)), C.ptr(eps),
               C.ptr(beta), C.ptr(pin), C.ptr(pout), C.ptr(y), self.directions, R, *geom,
               self.in_sparsity, self.out_sparsity, 1 if self.antithetic else 0, C.ptr(buf), nbytes, C.stream())
        return y


class Synthetic(Perturbed):
    """One shared noise tensor re-used by every member through per-member +-1 sign flips of the
    inputs and/or outputs (reference ``base.py:269-347``).  ``input_flips`` is ``(directions, in)``,
    ``output_flips`` ``(directions, out)``, both int8."""

    def __init__(self, in_degree, out_degree, directions, antithetic=False, options={}, flip="auto",
                 in_sparsity=0, out_sparsity=0):
        Perturbed.__init__(self, directions, antithetic, options)
        if flip == "auto":
            if 1 < in_degree < 32 and 1 < out_degree < 32:
                flip = "both"
            else:
                flip = "in" if in_degree > out_degree else "out"
        if flip not in ("in", "out", "both"):
            raise NotImplementedError("Flip setting not recognized")
        self.flip_inputs = flip != "out"
        self.flip_outputs = flip != "in"
        self.in_degree = in_degree
        self.out_degree = out_degree
        if in_sparsity or out_sparsity:
            raise NotImplementedError("Sparsity is not efficient for synthetic sampling, use permuted sampling instead")
        self.in_sparsity = in_degree
        self.out_sparsity = out_degree
        if options.get("combined") and self.flip_inputs and self.flip_outputs:
            raise NotImplementedError("Can't do combined multiplication with both input and output flips")

    def allocate_weight(self):
        self.weight_noise = torch.empty((self.out_sparsity, self.in_sparsity) + tuple(self.weight.shape[2:]),
                                        device=self.weight.device, dtype=self.weight.dtype)

    def free_memory(self):
        Perturbed.free_memory(self)
        self.input_flips = None
        self.output_flips = None

    def _sample_flips(self, n, stream_id):
        out = torch.empty((self.directions, n), dtype=torch.int8, device=self.weight.device)
        C.call("nes_fill_signs", C.ptr(out), out.numel(), (int(self.seed) * 4 + stream_id) & (2 ** 64 - 1),
               self._member_groups(self.member_offset, n, 128), C.stream())
        return out

    def set_noise(self, noise_scale=None):
        """Shared noise, bias noise and sign flips drawn on the device (reference ``base.py:311-328``)."""
        self._prepare_noise(noise_scale)
        self._fill_normal(self.weight_noise, self.noise_scale, self.seed, 0)
        if self.bias is not None:
            self._fill_normal(self.bias_noise, self.noise_scale, self.seed, 1, self.member_offset)
        if self.flip_outputs:
            self.output_flips = self._sample_flips(self.out_degree, 2)
        if self.flip_inputs:
            self.input_flips = self._sample_flips(self.in_degree, 3)

    def _flips(self):
        fin = C.require_cuda(self.input_flips, "input_flips", torch.int8) if self.flip_inputs else None
        fout = C.require_cuda(self.output_flips, "output_flips", torch.int8) if self.flip_outputs else None
        return fin, fout

    def _weight_grad_regularised(self, weights, l1, l2, out=None):
        """eps * sum_d w_d f_out[d] f_in[d]^T (reference ``base.py:338-347``; the reference's two-sided
        einsum multiplies by w_d twice, ``base.py:340`` -- here it is the plain fitness-weighted sum)."""
        eps = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        weights = C.require_cuda(weights, "weights", _F32)
        if weights.numel() != self.directions:
            raise RuntimeError("update weights must have one entry per direction")
        fin, fout = self._flips()
        ksize = 1
        for sdim in self.weight.shape[2:]:
            ksize *= sdim
        grad = out if out is not None else torch.empty_like(self.weight, memory_format=torch.contiguous_format)
        nbytes = C.call("nes_synthetic_update_scratch_bytes", self.in_degree, self.out_degree)
        buf = C.scratch(nbytes, eps.device)
        C.call("nes_synthetic_update", C.ptr(eps), C.ptr(weights), C.ptr(fin), C.ptr(fout),
               C.ptr(_opt(self.weight)) if (l1 or l2) else None, C.ptr(grad), self.directions, self.in_degree,
               self.out_degree, ksize, float(l1), float(l2), C.ptr(buf), nbytes, C.stream())
        return grad

    def weight_grad(self, weights):
        return self._weight_grad_regularised(weights, 0, 0)


class SyntheticLinear(nn.Linear, _LinearMixin, Synthetic):
    """``y = x W^T + b + s * (f_out * ((x * f_in) eps^T) + beta_d)`` (reference ``base.py:601-628``)."""

    def __init__(self, in_features, out_features, directions, bias=True, antithetic=False, options={},
                 flip="auto", in_sparsity=0, out_sparsity=0):
        nn.Linear.__init__(self, in_features, out_features, bias)
        Synthetic.__init__(self, in_features, out_features, directions, antithetic=antithetic, options=options,
                           flip=flip, in_sparsity=in_sparsity, out_sparsity=out_sparsity)

    def forward(self, input):
        if not self.perturbed_flag:
            return self._plain_forward(input)
        x, lead = self._flatten_rows(input)
        R = self._repeats(x.shape[0])
        eps = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        beta = C.require_cuda(self.bias_noise, "bias_noise", _F32) if self.bias is not None else None
        fin, fout = self._flips()
        y = torch.empty((x.shape[0], self.out_features), device=x.device, dtype=_F32)
        mode = self.options.get("tc", "3xtf32")
        if mode not in ("3xtf32", "tf32", "fp32"):
            raise NotImplementedError('options["tc"] must be "3xtf32", "tf32" or "fp32"')
        if mode != "fp32" and self.in_features % 4 == 0 and x.shape[0]:
            self.last_path = mode
            m = _TC_MODES[mode]
            nbytes = C.call("nes_synthetic_linear_fwd_tc_scratch_bytes", self.directions, R, self.in_features,
                            self.out_features, m)
            buf = C.scratch(nbytes, x.device)
            C.call("nes_synthetic_linear_fwd_tc", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)), C.ptr(eps),
                   C.ptr(beta), C.ptr(fin), C.ptr(fout), C.ptr(y), self.directions, R, self.in_features,
                   self.out_features, 1 if self.antithetic else 0, m, C.ptr(buf), nbytes, C.stream())
            return y.view(*lead, self.out_features)
        self.last_path = "fp32"
        nbytes = C.call("nes_synthetic_linear_fwd_scratch_bytes", self.directions, R, self.out_features)
        buf = C.scratch(nbytes, x.device)
        C.call("nes_synthetic_linear_fwd", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)), C.ptr(eps),
               C.ptr(beta), C.ptr(fin), C.ptr(fout), C.ptr(y), self.directions, R, self.in_features,
               self.out_features, 1 if self.antithetic else 0, C.ptr(buf), nbytes, C.stream())
        return y.view(*lead, self.out_features)


class SyntheticConv2d(nn.Conv2d, _ConvMixin, Synthetic):
    """Sign-flip sampling on channels (reference ``base.py:631-668``): per member a convolution with
    ``W + s * f_out[d,k] * f_in[d,c] * eps[k,c]``."""

    def __init__(self, in_channels, out_channels, kernel_size, directions, stride=1, padding=0, dilation=1,
                 groups=1, bias=True, antithetic=False, options={}, padding_mode='zeros', flip="auto",
                 in_sparsity=0, out_sparsity=0):
        nn.Conv2d.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups,
                           bias, padding_mode)
        Synthetic.__init__(self, in_channels, out_channels, directions, antithetic=antithetic, options=options,
                           flip=flip, in_sparsity=in_sparsity, out_sparsity=out_sparsity)

    def forward(self, input):
        if not self.perturbed_flag:
            return self._plain_forward(input)
        x = C.require_cuda(input, "input", _F32)
        x, geom, out_hw = self._geometry(x)
        R = self._repeats(x.shape[0])
        eps = C.require_cuda(self.weight_noise, "weight_noise", _F32)
        beta = C.require_cuda(self.bias_noise, "bias_noise", _F32) if self.bias is not None else None
        fin, fout = self._flips()
        y = torch.empty((x.shape[0], self.out_channels) + out_hw, device=x.device, dtype=_F32)
        C.call("nes_synthetic_conv2d_fwd", C.ptr(x), C.ptr(_opt(self.weight)), C.ptr(_opt(self.bias)), C.ptr(eps),
               C.ptr(beta), C.ptr(fin), C.ptr(fout), C.ptr(y), self.directions, R, *geom,
               1 if self.antithetic else 0, C.stream())
        return y


class PerturbedAffine(nn.Module, Perturbed):
    """Per-member scale and shift, stored "direct" (``weight_noise = weight + noise``; reference
    ``base.py:427-444``).  Forward, noise set-up and update all run in the library; the update subtracts the
    parameter row by row as the reference does."""

    def __init__(self, normalized_shape, directions, antithetic=False, options={"direct": True}):
        nn.Module.__init__(self)
        self.weight = nn.Parameter(torch.ones(normalized_shape))
        self.bias = nn.Parameter(torch.zeros(normalized_shape))
        if not options.get("direct"):
            raise NotImplementedError("Only direct is implemented")
        Perturbed.__init__(self, directions, antithetic=antithetic, options=options)

    def forward(self, input):
        scale, shift = (self.weight_noise, self.bias_noise) if self.perturbed_flag else (self.weight.detach(), self.bias.detach())
        x = C.require_cuda(input, "input", _F32)
        # scale / shift broadcast against the trailing dimensions of the input (the reference's `input * w + b`)
        shape = torch.broadcast_shapes(tuple(x.shape), tuple(scale.shape))
        if shape != tuple(x.shape):
            x = x.expand(shape).contiguous()
        tail = shape[len(shape) - scale.dim():] if scale.dim() else ()
        if tuple(scale.shape) != tuple(tail):
            scale, shift = scale.expand(tail).contiguous(), shift.expand(tail).contiguous()
        scale = C.require_cuda(scale, "scale", _F32)
        shift = C.require_cuda(shift, "shift", _F32)
        y = torch.empty(shape, device=x.device, dtype=_F32)
        C.call("nes_affine_fwd", C.ptr(x), C.ptr(scale), C.ptr(shift), C.ptr(y), y.numel(), max(scale.numel(), 1),
               C.stream())
        return y
