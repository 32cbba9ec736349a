"""CPU oracle for the fp32 perturbed-layer path.  TEST INFRASTRUCTURE ONLY.

This file restates, as plain functions over CPU torch tensors, the arithmetic of the
reference's ``modules/base.py`` (NESgpu).  It is a checker: only the tests, the smoke
check and the benchmark's CPU-baseline leg may import it.  The product package never
does; it fails loudly when its CUDA library is missing.

Parity status: pinned.  ``tests/golden/make_golden.py`` imports the reference's own
``modules/base.py`` on CPU, injects seeded noise / permutation tensors and stores the
reference's outputs; ``tests/test_oracle.py`` checks every function below against those
stored outputs.

Conventions (reference ``modules/base.py``):
  * batch row ``b = r * D + d``: ``input.view(-1, D, in)`` (base.py:357,368,490);
  * antithetic sign: rows with ``r >= (R + 1) // 2`` get ``-1`` (base.py:377-378,504-505,584-585);
  * the noise scale is already baked into the stored noise tensors (base.py:83,206).
"""
import torch
import torch.nn.functional as F


def antithetic_signs(repeat, antithetic, dtype=torch.float32):
    """+1 for the first ``(repeat+1)//2`` repeats, -1 for the rest (base.py:377-378)."""
    s = torch.ones(repeat, dtype=dtype)
    if antithetic:
        s[(repeat + 1) // 2:] = -1
    return s


# ----------------------------------------------------------------------------------
# IID noise: PerturbedLinear / PerturbedConv2d / Perturbed.update
# ----------------------------------------------------------------------------------

def perturbed_linear_forward(x, weight, bias, weight_noise, bias_noise, directions,
                             antithetic=False, direct=False):
    """PerturbedLinear.forward with the perturbed flag set (base.py:355-381).

    x (R*D, in); weight (out, in); weight_noise (D, out, in); bias_noise (D, out) or None.
    direct=True follows base.py:356-364 (noise tensors already hold W+E / b+beta; the
    result is returned as (R, D, out))."""
    D = directions
    xin = x.view(-1, D, x.shape[-1]).permute(1, 0, 2)           # (D, R, in)
    R = xin.shape[1]
    pert = torch.bmm(xin, weight_noise.permute(0, 2, 1))          # (D, R, out)
    if bias_noise is not None:
        pert = pert + bias_noise.view(D, 1, -1)
    pert = pert.permute(1, 0, 2)                                  # (R, D, out)
    if direct:
        return pert.contiguous()
    base = F.linear(x, weight, bias)
    pert = pert * antithetic_signs(R, antithetic).view(R, 1, 1)
    return (base.view_as(pert) + pert).reshape(base.shape)


def perturbed_conv2d_forward(x, weight, bias, weight_noise, bias_noise, directions,
                             stride=1, padding=0, dilation=1, antithetic=False):
    """PerturbedConv2d.forward, non-direct branch (base.py:410-425): the grouped-conv
    trick is equal to a per-member convolution with that member's own noise filter."""
    D = directions
    base = F.conv2d(x, weight, bias, stride, padding, dilation)
    B = x.shape[0]
    R = B // D
    xv = x.view(R, D * x.shape[1], *x.shape[-2:])
    bn = bias_noise.reshape(-1) if bias_noise is not None else None
    pert = F.conv2d(xv, weight_noise.view(-1, *weight.shape[1:]), bn, stride, padding,
                    dilation, D)
    pert = pert.view(R, D, weight.shape[0], *pert.shape[-2:])
    pert = pert * antithetic_signs(R, antithetic).view(R, 1, 1, 1, 1)
    return base + pert.reshape(base.shape)


def perturbed_weight_grad(weight_noise, weights):
    """Perturbed.weight_grad (base.py:110-118): ``weights @ noise.view(D, -1)``."""
    D = weight_noise.shape[0]
    return (weights @ weight_noise.reshape(D, -1)).view(weight_noise.shape[1:])


def perturbed_update(weight, weight_noise, bias_noise, weights, l1=0.0, l2=0.0):
    """Perturbed.update (base.py:120-138) without the ``.grad`` accumulation: returns
    (grad, bias_grad or None)."""
    grad = perturbed_weight_grad(weight_noise, weights)
    if l1:
        grad = grad + l1 * torch.sign(weight)
    if l2:
        grad = grad + l2 * weight
    bias_grad = None
    if bias_noise is not None:
        bias_grad = weights @ bias_noise.reshape(bias_noise.shape[0], -1)
    return grad, bias_grad


# ----------------------------------------------------------------------------------
# Shared noise + per-member permutations: PermutedLinear / PermutedConv2d
# ----------------------------------------------------------------------------------

def resolve_permutation(in_degree, out_degree, permutation="auto", in_sparsity=0, out_sparsity=0):
    """Constructor rule of Permuted (base.py:148-184).  Returns
    (permute_inputs, permute_outputs, in_sparsity, out_sparsity)."""
    if permutation == "auto":
        if in_sparsity:
            permutation = "both" if out_sparsity else "in"
        elif out_sparsity:
            permutation = "out"
        elif 1 < in_degree < 32 and 1 < out_degree < 32:
            permutation = "both"
        elif in_degree > out_degree:
            permutation = "in"
        else:
            permutation = "out"
    if permutation not in ("both", "in", "out"):
        raise NotImplementedError("Permutation setting not recognized")
    p_in = permutation in ("both", "in")
    p_out = permutation in ("both", "out")
    if isinstance(in_sparsity, float):
        in_sparsity = max(1, int(in_sparsity * in_degree))
    if in_sparsity:
        p_in = True
    else:
        in_sparsity = in_degree
    if isinstance(out_sparsity, float):
        out_sparsity = max(1, int(out_sparsity * out_degree))
    if out_sparsity:
        p_out = True
    else:
        out_sparsity = out_degree
    return p_in, p_out, in_sparsity, out_sparsity


def gather_inputs(xv, input_permutations, in_degree):
    """Permuted.apply_input_permutation (base.py:229-233) on a (R, D*in, ...) view."""
    if input_permutations is None:
        return xv
    D = input_permutations.shape[0]
    idx = (input_permutations.long() + (torch.arange(D) * in_degree).unsqueeze(1)).flatten()
    return torch.index_select(xv, 1, idx)


def gather_outputs(pv, output_permutations, out_degree):
    """Permuted.apply_output_permutation (base.py:236-240) on a (R, D*out, ...) view."""
    if output_permutations is None:
        return pv
    D = output_permutations.shape[0]
    idx = (output_permutations.long() + (torch.arange(D) * out_degree).unsqueeze(1)).flatten()
    return torch.index_select(pv, 1, idx)


def permuted_linear_forward(x, weight, bias, weight_noise, bias_noise, input_permutations,
                            output_permutations, directions, antithetic=False):
    """PermutedLinear.forward, default (non-combined) branch (base.py:487-508).

    weight_noise (out_sp, in_sp); input_permutations (D, in_sp) or None;
    output_permutations (D, out) or None."""
    D = directions
    out_f, in_f = weight.shape
    out_sp, in_sp = weight_noise.shape
    base = F.linear(x, weight, bias)
    xv = x.view(-1, D * in_f)
    R = xv.shape[0]
    xg = gather_inputs(xv, input_permutations, in_f).reshape(-1, in_sp)
    pert = torch.zeros(R * D, out_f, dtype=x.dtype)
    pert[:, :out_sp] = xg @ weight_noise.t()
    q = gather_outputs(pert.view(R, D * out_f), output_permutations, out_f).view(R, D, out_f)
    if bias_noise is not None:
        q = q + bias_noise
    q = q * antithetic_signs(R, antithetic).view(R, 1, 1)
    return base + q.reshape(base.shape)


def permuted_conv2d_forward(x, weight, bias, weight_noise, bias_noise, input_permutations,
                            output_permutations, directions, stride=1, padding=0, dilation=1,
                            antithetic=False):
    """PermutedConv2d.forward, default branch (base.py:557-588).  The reference's bias-noise
    broadcast (base.py:583) only type-checks for R == 1; here it is applied per member for
    any R, which is what that line computes when R == 1."""
    D = directions
    out_c, in_c = weight.shape[:2]
    out_sp, in_sp = weight_noise.shape[:2]
    base = F.conv2d(x, weight, bias, stride, padding, dilation)
    R = x.shape[0] // D
    xv = x.view(R, D * in_c, *x.shape[-2:])
    xg = gather_inputs(xv, input_permutations, in_c).reshape(R * D, in_sp, *x.shape[-2:])
    pert = torch.zeros_like(base)
    pert[:, :out_sp] = F.conv2d(xg, weight_noise, None, stride, padding, dilation)
    q = gather_outputs(pert.view(R, D * out_c, *pert.shape[-2:]), output_permutations, out_c)
    q = q.reshape(R, D, out_c, *base.shape[-2:])
    if bias_noise is not None:
        q = q + bias_noise.view(1, D, out_c, 1, 1)
    q = q * antithetic_signs(R, antithetic).view(R, 1, 1, 1, 1)
    return base + q.reshape(base.shape)


def permutation_weights(weights, input_permutations, output_permutations, in_degree,
                        out_degree, in_sp, out_sp):
    """Permuted.get_permutation_weights for the single-sided modes (base.py:254-267):
    in-only  -> H (in_sp, in):   H[j, m] = sum_d w_d [pi_in[d, j] == m]
    out-only -> G (out, out_sp): G[k, s] = sum_d w_d [pi_out[d, k] == s], s < out_sp."""
    if input_permutations is not None and output_permutations is not None:
        raise ValueError("two-sided mode: use dense_member_noise")
    if input_permutations is not None:
        H = torch.zeros(in_sp, in_degree, dtype=weights.dtype)
        idx = input_permutations.long() + torch.arange(in_sp) * in_degree
        H.put_(idx, weights.view(-1, 1).expand(-1, in_sp), accumulate=True)
        return H
    G = torch.zeros(out_degree, out_degree, dtype=weights.dtype)
    idx = output_permutations.long() + torch.arange(out_degree) * out_degree
    G.put_(idx, weights.view(-1, 1).expand(-1, out_degree), accumulate=True)
    return G[:, :out_sp]


def permuted_linear_weight_grad(weight_noise, weights, input_permutations, output_permutations,
                                in_degree, out_degree):
    """PermutedLinear.weight_grad (base.py:511-518).  The two-sided case is evaluated as
    sum_d w_d E_d with the dense member noise, which is what base.py:243-253,514 computes
    where the reference is self-consistent (in_sp == in)."""
    out_sp, in_sp = weight_noise.shape[:2]
    if input_permutations is not None and output_permutations is not None:
        E = dense_member_noise(weight_noise, input_permutations, output_permutations,
                               in_degree, out_degree)
        return torch.einsum("d,dkm->km", weights, E)
    pw = permutation_weights(weights, input_permutations, output_permutations, in_degree,
                             out_degree, in_sp, out_sp)
    if input_permutations is not None:
        return weight_noise @ pw
    return pw @ weight_noise


def permuted_conv2d_weight_grad(weight_noise, weights, input_permutations, output_permutations,
                                in_degree, out_degree):
    """PermutedConv2d.weight_grad (base.py:590-599)."""
    out_sp, in_sp, kh, kw = weight_noise.shape
    if input_permutations is not None and output_permutations is not None:
        E = dense_member_noise(weight_noise, input_permutations, output_permutations,
                               in_degree, out_degree)
        return torch.einsum("d,dkmij->kmij", weights, E)
    pw = permutation_weights(weights, input_permutations, output_permutations, in_degree,
                             out_degree, in_sp, out_sp)
    if input_permutations is not None:
        g = weight_noise.permute(0, 2, 3, 1).reshape(-1, in_sp) @ pw
        return g.view(out_sp, kh, kw, in_degree).permute(0, 3, 1, 2).contiguous()
    return (pw @ weight_noise.reshape(out_sp, -1)).view(out_degree, in_sp, kh, kw)


def dense_member_noise(weight_noise, input_permutations, output_permutations, in_degree,
                       out_degree):
    """The dense per-member noise a Permuted layer is equal to:
    E_d[k, m, ...] = sum_j [pi_in[d, j] == m] * eps_pad[pi_out[d, k], j, ...]
    with eps zero-padded to ``out`` rows.  Derived from base.py:487-508 / 557-588; used for
    size-independent property tests and for the two-sided update."""
    out_sp, in_sp = weight_noise.shape[:2]
    tail = weight_noise.shape[2:]
    D = (input_permutations if input_permutations is not None else output_permutations).shape[0]
    eps_pad = torch.zeros(out_degree, in_sp, *tail, dtype=weight_noise.dtype)
    eps_pad[:out_sp] = weight_noise
    E = torch.zeros(D, out_degree, in_degree, *tail, dtype=weight_noise.dtype)
    for d in range(D):
        rows = eps_pad if output_permutations is None else eps_pad[output_permutations[d].long()]
        if input_permutations is None:
            E[d] = rows
        else:
            E[d].index_add_(1, input_permutations[d].long(), rows)
    return E


# ----------------------------------------------------------------------------------
# Shared noise + per-member sign flips: SyntheticLinear / SyntheticConv2d
# ----------------------------------------------------------------------------------

def synthetic_linear_forward(x, weight, bias, weight_noise, bias_noise, input_flips, output_flips, directions,
                             antithetic=False):
    """SyntheticLinear.forward (base.py:611-628).  input_flips (D, in) / output_flips (D, out), +-1, or None."""
    D = directions
    base = F.linear(x, weight, bias)
    xv = x.view(-1, D, x.shape[-1])
    R = xv.shape[0]
    fx = xv * input_flips if input_flips is not None else xv
    pert = fx @ weight_noise.t()
    if output_flips is not None:
        pert = pert * output_flips
    if bias_noise is not None:
        pert = pert + bias_noise
    pert = pert * antithetic_signs(R, antithetic).view(R, 1, 1)
    return base + pert.reshape(base.shape)


def synthetic_conv2d_forward(x, weight, bias, weight_noise, bias_noise, input_flips, output_flips, directions,
                             stride=1, padding=0, dilation=1, antithetic=False):
    """SyntheticConv2d.forward (base.py:642-668)."""
    D = directions
    base = F.conv2d(x, weight, bias, stride, padding, dilation)
    R = x.shape[0] // D
    xv = x.view(R, D, *x.shape[1:])
    fx = xv * input_flips.view(1, D, -1, 1, 1) if input_flips is not None else xv
    pert = F.conv2d(fx.reshape(x.shape), weight_noise, None, stride, padding, dilation)
    pert = pert.view(R, D, *pert.shape[1:])
    if output_flips is not None:
        pert = pert * output_flips.view(1, D, -1, 1, 1)
    if bias_noise is not None:
        pert = pert + bias_noise.view(1, D, -1, 1, 1)
    pert = pert * antithetic_signs(R, antithetic).view(R, 1, 1, 1, 1)
    return base + pert.reshape(base.shape)


def synthetic_weight_grad(weight_noise, weights, input_flips, output_flips):
    """Synthetic.weight_grad for the one-sided modes (base.py:343-347), and sum_d w_d E_d for two-sided
    flips (the reference's two-sided einsum, base.py:340, multiplies by w_d twice; that is not followed)."""
    nd = weight_noise.dim()
    if input_flips is not None and output_flips is not None:
        fw = torch.einsum("d,da,db->ab", weights, output_flips.float(), input_flips.float())
        return fw.view(*fw.shape, *[1] * (nd - 2)) * weight_noise
    if input_flips is not None:
        fw = (input_flips.float() * weights.unsqueeze(1)).sum(dim=0)
        return fw.view(1, -1, *[1] * (nd - 2)) * weight_noise
    fw = (output_flips.float() * weights.unsqueeze(1)).sum(dim=0)
    return fw.view(-1, *[1] * (nd - 1)) * weight_noise


# ----------------------------------------------------------------------------------
# Sparse Gaussian noise (README.md:12,29-30; no source in the reference snapshot)
# ----------------------------------------------------------------------------------

def densify_sparse_noise(indices, values, in_features):
    """(D, out, k) index/value pairs -> dense (D, out, in) noise; duplicate indices add."""
    D, out_f, _ = indices.shape
    E = torch.zeros(D, out_f, in_features, dtype=values.dtype)
    E.scatter_add_(2, indices.long(), values)
    return E


def sparse_perturbed_linear_forward(x, weight, bias, indices, values, bias_noise, directions,
                                    antithetic=False):
    """SparsePerturbedLinear is defined as PerturbedLinear (base.py:365-381) applied to the
    densified noise; parity for this layer is therefore pinned through perturbed_linear_forward."""
    E = densify_sparse_noise(indices, values, weight.shape[1])
    return perturbed_linear_forward(x, weight, bias, E, bias_noise, directions, antithetic)


# ----------------------------------------------------------------------------------
# Fitness shaping used by the benchmark configurations (not part of the reference layers)
# ----------------------------------------------------------------------------------

def centered_ranks(fitness):
    """rank / (n - 1) - 1/2 with a stable argsort."""
    n = fitness.numel()
    order = torch.argsort(fitness, stable=True)
    ranks = torch.empty(n, dtype=torch.float32)
    ranks[order] = torch.arange(n, dtype=torch.float32)
    return ranks / (n - 1) - 0.5
