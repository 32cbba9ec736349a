"""Generates the golden vectors under tests/golden/ from the reference itself.

Run once, where a checkout of the reference is available; pass its root as the first argument (or set
``NES_REFERENCE_ROOT``):

    python tests/golden/make_golden.py <reference checkout>

fp32 layers: the reference's own ``modules/base.py`` is imported on CPU, its layers are
constructed at small shapes, the noise / permutation tensors are assigned (bypassing
``set_noise``) and ``forward`` / ``update`` / ``get_permutation_weights`` are executed; the
inputs, the injected tensors and the reference's outputs are stored in
``perturbed_golden.npz``.

binary ops: the reference's bit kernels need cupy and a GPU, so its results cannot be
produced here.  ``binary_golden.npz`` instead holds the *naive formulas* the reference's
own check script compares its kernels with (``booloptests.py:94-95,138-141,150-160``):
a grouped +-1 convolution with -1 padding, ``2*conv > thresh`` and ``F.max_pool2d`` on the
unpacked bits, evaluated with CPU torch on seeded random bits.
"""
import json
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    return None if t is None else t.detach().cpu().numpy()


def _perms(gen, D, n, keep=None, repeats=False):
    if repeats:
        return torch.randint(n, (D, keep or n), generator=gen).short()
    p = torch.stack([torch.randperm(n, generator=gen) for _ in range(D)]).short()
    return p[:, :keep] if keep else p


def perturbed_cases(base):
    gen = torch.Generator().manual_seed(20240)
    out = {}
    meta = {}

    def rnd(*shape, scale=1.0):
        return torch.randn(*shape, generator=gen) * scale

    def record(name, kw, tensors):
        meta[name] = kw
        for k, v in tensors.items():
            if v is not None:
                out[f"{name}/{k}"] = _np(v)

    # ---- PerturbedLinear (base.py:349-381) and Perturbed.update (base.py:120-138)
    for name, D, R, in_f, out_f, anti, bias, direct in [
        ("plin_a", 6, 2, 24, 20, True, True, False),
        ("plin_b", 5, 3, 17, 9, True, True, False),
        ("plin_c", 4, 1, 8, 12, False, False, False),
        ("plin_direct", 4, 2, 10, 7, False, True, True),
    ]:
        layer = base.PerturbedLinear(in_f, out_f, D, bias=bias, antithetic=anti,
                                     options={"direct": True} if direct else {})
        layer.weight_noise = rnd(D, out_f, in_f, scale=0.1)
        if direct:
            layer.weight_noise = layer.weight_noise + layer.weight.detach()
        if bias:
            layer.bias_noise = rnd(D, out_f, scale=0.1)
            if direct:
                layer.bias_noise = layer.bias_noise + layer.bias.detach()
        x = rnd(R * D, in_f)
        w = rnd(D)
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(x)
            layer.perturbed_flag = False
            y_off = layer.forward(x)
            upd = layer.update(w, l1=0.01, l2=0.02)
        grad, bgrad = upd if bias else (upd, None)
        record(name, dict(kind="PerturbedLinear", D=D, R=R, in_f=in_f, out_f=out_f, antithetic=anti,
                          bias=bias, direct=direct, l1=0.01, l2=0.02),
               dict(x=x, weight=layer.weight, bias=layer.bias, weight_noise=layer.weight_noise,
                    bias_noise=layer.bias_noise if bias else None, w=w, y=y, y_off=y_off,
                    grad=grad, bias_grad=bgrad))

    # ---- PerturbedConv2d (base.py:384-425)
    for name, D, R, cin, cout, k, hw, stride, pad, anti in [
        ("pconv_a", 4, 2, 3, 5, 3, 8, 1, 1, True),
        ("pconv_b", 3, 1, 2, 4, 3, 9, 2, 0, False),
    ]:
        layer = base.PerturbedConv2d(cin, cout, k, D, stride=stride, padding=pad, antithetic=anti)
        layer.weight_noise = rnd(D, cout, cin, k, k, scale=0.1)
        layer.bias_noise = rnd(D, cout, scale=0.1)
        x = rnd(R * D, cin, hw, hw)
        w = rnd(D)
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(x)
            layer.perturbed_flag = False
            grad, bgrad = layer.update(w)
        record(name, dict(kind="PerturbedConv2d", D=D, R=R, cin=cin, cout=cout, k=k, hw=hw,
                          stride=stride, padding=pad, antithetic=anti),
               dict(x=x, weight=layer.weight, bias=layer.bias, weight_noise=layer.weight_noise,
                    bias_noise=layer.bias_noise, w=w, y=y, grad=grad, bias_grad=bgrad))

    # ---- PermutedLinear (base.py:447-518) incl. get_permutation_weights (base.py:242-267)
    for name, D, R, in_f, out_f, anti, mode, in_sp, out_sp, repeats in [
        ("permlin_out", 6, 2, 16, 12, True, "out", 0, 0, False),
        ("permlin_in", 5, 2, 20, 8, True, "in", 0, 0, False),
        ("permlin_both", 4, 3, 6, 5, True, "both", 0, 0, False),
        ("permlin_out_sp", 6, 1, 10, 16, False, "out", 0, 0.5, False),
        ("permlin_in_sp", 7, 2, 30, 6, False, "in", 0.3, 0, False),
        ("permlin_auto_sp_both", 4, 2, 12, 10, True, "auto", 0.5, 0.5, False),
        ("permlin_in_repeats", 5, 2, 14, 6, False, "in", 5, 0, True),
    ]:
        layer = base.PermutedLinear(in_f, out_f, D, antithetic=anti, permutation=mode,
                                    in_sparsity=in_sp, out_sparsity=out_sp)
        osp, isp = layer.out_sparsity, layer.in_sparsity
        layer.weight_noise = rnd(osp, isp, scale=0.1)
        layer.bias_noise = rnd(D, out_f, scale=0.1)
        layer.input_permutations = _perms(gen, D, in_f, isp, repeats) if layer.permute_inputs else None
        layer.output_permutations = _perms(gen, D, out_f) if layer.permute_outputs else None
        x = rnd(R * D, in_f)
        w = rnd(D)
        two_sided = layer.permute_inputs and layer.permute_outputs
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(x)
            layer.perturbed_flag = False
            pw = grad = bgrad = None
            if not (two_sided and isp < in_f):   # base.py:248 is wrong when in_sp < in
                pw = layer.get_permutation_weights(w)
                grad, bgrad = layer.update(w)
            else:
                bgrad = w @ layer.bias_noise
        record(name, dict(kind="PermutedLinear", D=D, R=R, in_f=in_f, out_f=out_f, antithetic=anti,
                          permute_inputs=layer.permute_inputs, permute_outputs=layer.permute_outputs,
                          in_sp=isp, out_sp=osp, mode=mode, in_sparsity=in_sp, out_sparsity=out_sp),
               dict(x=x, weight=layer.weight, bias=layer.bias, weight_noise=layer.weight_noise,
                    bias_noise=layer.bias_noise, pin=layer.input_permutations,
                    pout=layer.output_permutations, w=w, y=y,
                    perm_weights=None if (pw is None or two_sided) else pw.contiguous(),
                    grad=grad, bias_grad=bgrad))

    # ---- PermutedConv2d (base.py:521-599); R == 1 because of the bias-noise broadcast (base.py:583)
    for name, D, cin, cout, k, hw, stride, pad, anti, mode, in_sp, out_sp in [
        ("permconv_out_sp", 6, 4, 8, 3, 8, 1, 1, False, "auto", 0, 0.5),
        ("permconv_in", 5, 6, 3, 3, 7, 1, 1, False, "in", 0, 0),
        ("permconv_both", 4, 3, 4, 3, 6, 2, 1, False, "both", 0, 0),
        ("permconv_in_sp", 4, 8, 4, 1, 5, 1, 0, False, "auto", 0.5, 0),
    ]:
        layer = base.PermutedConv2d(cin, cout, k, D, stride=stride, padding=pad, antithetic=anti,
                                    permutation=mode, in_sparsity=in_sp, out_sparsity=out_sp)
        osp, isp = layer.out_sparsity, layer.in_sparsity
        layer.weight_noise = rnd(osp, isp, k, k, scale=0.1)
        layer.bias_noise = rnd(D, cout, scale=0.1)
        layer.input_permutations = _perms(gen, D, cin, isp) if layer.permute_inputs else None
        layer.output_permutations = _perms(gen, D, cout) if layer.permute_outputs else None
        x = rnd(D, cin, hw, hw)
        w = rnd(D)
        two_sided = layer.permute_inputs and layer.permute_outputs
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(x)
            layer.perturbed_flag = False
            grad, bgrad = layer.update(w)
        record(name, dict(kind="PermutedConv2d", D=D, R=1, cin=cin, cout=cout, k=k, hw=hw,
                          stride=stride, padding=pad, antithetic=anti,
                          permute_inputs=layer.permute_inputs, permute_outputs=layer.permute_outputs,
                          in_sp=isp, out_sp=osp, mode=mode, in_sparsity=in_sp, out_sparsity=out_sp),
               dict(x=x, weight=layer.weight, bias=layer.bias, weight_noise=layer.weight_noise,
                    bias_noise=layer.bias_noise, pin=layer.input_permutations,
                    pout=layer.output_permutations, w=w, y=y, grad=grad.contiguous(), bias_grad=bgrad))

    # ---- SyntheticLinear / SyntheticConv2d (base.py:269-347, 601-668); one-sided updates only for the
    # stored gradient (the two-sided einsum at base.py:340 squares the weights)
    for name, D, R, in_f, out_f, anti, flip in [
        ("synlin_in", 5, 2, 18, 7, True, "in"), ("synlin_out", 6, 3, 9, 14, True, "out"),
        ("synlin_both", 4, 2, 6, 5, False, "both"), ("synlin_auto", 4, 1, 40, 8, False, "auto"),
    ]:
        layer = base.SyntheticLinear(in_f, out_f, D, antithetic=anti, flip=flip)
        layer.weight_noise = rnd(out_f, in_f, scale=0.1)
        layer.bias_noise = rnd(D, out_f, scale=0.1)
        layer.input_flips = (2 * torch.randint(2, (D, in_f), generator=gen) - 1).to(torch.int8) if layer.flip_inputs else None
        layer.output_flips = (2 * torch.randint(2, (D, out_f), generator=gen) - 1).to(torch.int8) if layer.flip_outputs else None
        x = rnd(R * D, in_f)
        w = rnd(D)
        two_sided = layer.flip_inputs and layer.flip_outputs
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(x)
            layer.perturbed_flag = False
            grad = None if two_sided else layer.weight_grad(w).contiguous()
        record(name, dict(kind="SyntheticLinear", D=D, R=R, in_f=in_f, out_f=out_f, antithetic=anti, flip=flip,
                          flip_inputs=layer.flip_inputs, flip_outputs=layer.flip_outputs),
               dict(x=x, weight=layer.weight, bias=layer.bias, weight_noise=layer.weight_noise,
                    bias_noise=layer.bias_noise, fin=layer.input_flips, fout=layer.output_flips, w=w, y=y, grad=grad))
    for name, D, R, cin, cout, k, hw, stride, pad, anti, flip in [
        ("synconv_in", 4, 1, 6, 3, 3, 7, 1, 1, False, "in"), ("synconv_out", 3, 1, 2, 5, 3, 8, 2, 1, False, "out"),   # R == 1: base.py:661,663 broadcast
        ("synconv_both", 4, 1, 3, 4, 1, 5, 1, 0, False, "both"),
    ]:
        layer = base.SyntheticConv2d(cin, cout, k, D, stride=stride, padding=pad, antithetic=anti, flip=flip)
        layer.weight_noise = rnd(cout, cin, k, k, scale=0.1)
        layer.bias_noise = rnd(D, cout, scale=0.1)
        layer.input_flips = (2 * torch.randint(2, (D, cin), generator=gen) - 1).to(torch.int8) if layer.flip_inputs else None
        layer.output_flips = (2 * torch.randint(2, (D, cout), generator=gen) - 1).to(torch.int8) if layer.flip_outputs else None
        x = rnd(R * D, cin, hw, hw)
        w = rnd(D)
        two_sided = layer.flip_inputs and layer.flip_outputs
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(x)
            layer.perturbed_flag = False
            grad = None if two_sided else layer.weight_grad(w).contiguous()
        record(name, dict(kind="SyntheticConv2d", D=D, R=R, cin=cin, cout=cout, k=k, hw=hw, stride=stride, padding=pad,
                          antithetic=anti, flip=flip, flip_inputs=layer.flip_inputs, flip_outputs=layer.flip_outputs),
               dict(x=x, weight=layer.weight, bias=layer.bias, weight_noise=layer.weight_noise,
                    bias_noise=layer.bias_noise, fin=layer.input_flips, fout=layer.output_flips, w=w, y=y, grad=grad))

    # ---- PerturbedAffine (base.py:427-444), direct storage
    D, shape = 5, (7,)
    layer = base.PerturbedAffine(shape, D)
    with torch.no_grad():
        layer.weight.copy_(rnd(*shape) + 1)
        layer.bias.copy_(rnd(*shape))
    layer.weight_noise = rnd(D, *shape, scale=0.1) + layer.weight.detach()
    layer.bias_noise = rnd(D, *shape, scale=0.1) + layer.bias.detach()
    x = rnd(3, D, *shape)
    w = rnd(D)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(x)
        layer.perturbed_flag = False
        grad, bgrad = layer.update(w)
    record("affine", dict(kind="PerturbedAffine", D=D, shape=list(shape)),
           dict(x=x, weight=layer.weight, bias=layer.bias, weight_noise=layer.weight_noise,
                bias_noise=layer.bias_noise, w=w, y=y, grad=grad, bias_grad=bgrad))

    # ---- constructor rule of Permuted (base.py:148-184)
    rules = []
    for in_d, out_d, mode, isp, osp in [
        (256, 256, "auto", 0, 0), (1600, 128, "auto", 0, 0), (8, 8, "auto", 0, 0),
        (64, 64, "auto", 0, 0.5), (64, 64, "auto", 0.1, 0), (64, 64, "auto", 0.1, 0.9),
        (10, 300, "in", 0, 7), (10, 300, "out", 3, 0), (5, 5, "both", 0, 0), (100, 100, "auto", 0.001, 0),
    ]:
        layer = base.PermutedLinear(in_d, out_d, 2, permutation=mode, in_sparsity=isp, out_sparsity=osp)
        rules.append(dict(args=[in_d, out_d, mode, isp, osp],
                          result=[layer.permute_inputs, layer.permute_outputs,
                                  layer.in_sparsity, layer.out_sparsity]))
    meta["__constructor_rules__"] = rules
    return out, meta


def binary_cases():
    gen = torch.Generator().manual_seed(777)
    out = {}
    meta = {}
    for name, P, cin, cout, size, f, pad, stride in [
        ("bconv_f1", 5, 64, 6, 6, 1, 0, 1),
        ("bconv_f3", 4, 70, 5, 7, 3, 1, 1),
        ("bconv_f3s2", 3, 33, 4, 9, 3, 2, 2),
        ("bconv_f7", 2, 8, 3, 10, 7, 2, 3),
    ]:
        inp = torch.randint(2, (P, size, size, cin), generator=gen).bool()
        filt = torch.randint(2, (P, cout, f, f, cin), generator=gen).bool()
        n = f * f * cin
        thresh = torch.randint(n, (P, cout), generator=gen).int() - n // 2 + n
        # booloptests.py:150-160: inputs 2(b-.5), filters -2(b-.5), pad value -1, grouped conv
        ni = (2 * (inp.float() - .5)).permute(0, 3, 1, 2).reshape(1, P * cin, size, size)
        nf = (-2 * (filt.float() - .5)).permute(0, 1, 4, 2, 3).reshape(P * cout, cin, f, f)
        res = torch.conv2d(F.pad(ni, (pad,) * 4, value=-1), nf, stride=(stride, stride), groups=P)
        res = res.view(P, cout, *res.shape[-2:]).permute(0, 2, 3, 1).round().int()
        conv_counts = (res + n) // 2                      # 2*conv - n == naive  (booloptests.py:160)
        act = 2 * conv_counts > thresh.view(P, 1, 1, cout)  # booloptests.py:157-159
        # booloptests.py:94-95,138-141: 2x2/stride-2 max-pool of the bits
        mp = F.max_pool2d(inp.permute(0, 3, 1, 2).float(), (2, 2), (2, 2), (0, 0)).permute(0, 2, 3, 1).bool()
        meta[name] = dict(P=P, cin=cin, cout=cout, size=size, f=f, pad=pad, stride=stride)
        for k, v in dict(inp=inp, filt=filt, thresh=thresh, conv_counts=conv_counts, act=act,
                         maxpool=mp).items():
            out[f"{name}/{k}"] = _np(v)
    return out, meta


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NES_REFERENCE_ROOT")
    if not ref_root or not os.path.isdir(ref_root):
        raise SystemExit("usage: make_golden.py <reference checkout>  (or set NES_REFERENCE_ROOT)")
    sys.path.insert(0, ref_root)
    import modules.base as base   # the reference's own file
    torch.manual_seed(0)
    arrays, meta = perturbed_cases(base)
    np.savez_compressed(os.path.join(HERE, "perturbed_golden.npz"), __meta__=json.dumps(meta), **arrays)
    arrays, meta = binary_cases()
    np.savez_compressed(os.path.join(HERE, "binary_golden.npz"), __meta__=json.dumps(meta), **arrays)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
