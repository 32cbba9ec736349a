"""GPU parity of the fp32 perturbed layers (through the layer API -> ctypes -> C ABI) against
the golden vectors produced by the reference and against the CPU oracle on seeded inputs."""
import numpy as np
import pytest
import torch

from gpu_util import DEV, G, T, assert_close, set_params
from oracle import perturbed_ref as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def base():
    from nesgpu_b200 import base as b
    return b


def gen(seed):
    return torch.Generator().manual_seed(seed)


def perms(g, D, n, keep=None):
    p = torch.stack([torch.randperm(n, generator=g) for _ in range(D)]).short()
    return p[:, :keep].contiguous() if keep else p


# ------------------------------------------------------------------ golden vectors

def test_golden_perturbed_linear(base, perturbed_golden):
    for name in perturbed_golden.names("PerturbedLinear"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        layer = base.PerturbedLinear(m["in_f"], m["out_f"], m["D"], bias=m["bias"], antithetic=m["antithetic"],
                                     options={"direct": True} if m["direct"] else {}).to(DEV)
        set_params(layer, c["weight"], c.get("bias"))
        layer.weight_noise = G(c["weight_noise"])
        if m["bias"]:
            layer.bias_noise = G(c["bias_noise"])
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(G(c["x"]))
            layer.perturbed_flag = False
            y_off = layer.forward(G(c["x"]))
            upd = layer.update(G(c["w"]), l1=m["l1"], l2=m["l2"])
        assert_close(y, c["y"], what=name + " forward")
        assert_close(y_off, c["y_off"], what=name + " inference")
        grad, bgrad = upd if m["bias"] else (upd, None)
        assert_close(grad, c["grad"], what=name + " grad")
        assert layer.weight.grad is grad
        if m["bias"]:
            assert_close(bgrad, c["bias_grad"], what=name + " bias grad")
        # second update accumulates into .grad (base.py:126)
        with torch.no_grad():
            layer.update(G(c["w"]), l1=m["l1"], l2=m["l2"])
        assert_close(layer.weight.grad, 2 * T(c["grad"]), what=name + " accumulated grad")


def test_golden_perturbed_conv(base, perturbed_golden):
    for name in perturbed_golden.names("PerturbedConv2d"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        layer = base.PerturbedConv2d(m["cin"], m["cout"], m["k"], m["D"], stride=m["stride"],
                                     padding=m["padding"], antithetic=m["antithetic"]).to(DEV)
        set_params(layer, c["weight"], c["bias"])
        layer.weight_noise = G(c["weight_noise"])
        layer.bias_noise = G(c["bias_noise"])
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(G(c["x"]))
            layer.perturbed_flag = False
            grad, bgrad = layer.update(G(c["w"]))
        assert_close(y, c["y"], what=name + " forward")
        assert_close(grad, c["grad"], what=name + " grad")
        assert_close(bgrad, c["bias_grad"], what=name + " bias grad")


def _permuted_layer(base, cls, m, c, **kw):
    layer = cls(antithetic=m["antithetic"], permutation=m["mode"], in_sparsity=m["in_sparsity"],
                out_sparsity=m["out_sparsity"], **kw).to(DEV)
    assert (layer.permute_inputs, layer.permute_outputs, layer.in_sparsity, layer.out_sparsity) == \
        (m["permute_inputs"], m["permute_outputs"], m["in_sp"], m["out_sp"])
    set_params(layer, c["weight"], c["bias"])
    layer.weight_noise = G(c["weight_noise"])
    layer.bias_noise = G(c["bias_noise"])
    layer.input_permutations = G(c.get("pin"))
    layer.output_permutations = G(c.get("pout"))
    return layer


def test_golden_permuted_linear(base, perturbed_golden):
    for name in perturbed_golden.names("PermutedLinear"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        layer = _permuted_layer(base, lambda **kw: base.PermutedLinear(m["in_f"], m["out_f"], m["D"], **kw), m, c)
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(G(c["x"]))
            layer.perturbed_flag = False
            grad, bgrad = layer.update(G(c["w"]))
        assert_close(y, c["y"], what=name + " forward")
        assert_close(bgrad, c["bias_grad"], what=name + " bias grad")
        if "grad" in c:
            assert_close(grad, c["grad"], what=name + " grad")
        else:   # the reference's own two-sided update is wrong for in_sp < in: check against sum_d w_d E_d
            E = O.dense_member_noise(T(c["weight_noise"]), T(c.get("pin")), T(c.get("pout")), m["in_f"], m["out_f"])
            assert_close(grad, torch.einsum("d,dkm->km", T(c["w"]), E), what=name + " grad (dense form)")
        if "perm_weights" in c:
            with torch.no_grad():
                pw = layer.get_permutation_weights(G(c["w"]))
            assert_close(pw, c["perm_weights"], what=name + " permutation weights")


def test_golden_permuted_conv(base, perturbed_golden):
    for name in perturbed_golden.names("PermutedConv2d"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        layer = _permuted_layer(base, lambda **kw: base.PermutedConv2d(m["cin"], m["cout"], m["k"], m["D"],
                                                                       stride=m["stride"], padding=m["padding"], **kw), m, c)
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(G(c["x"]))
            layer.perturbed_flag = False
            grad, bgrad = layer.update(G(c["w"]))
        assert_close(y, c["y"], what=name + " forward")
        assert_close(grad, c["grad"], what=name + " grad")
        assert_close(bgrad, c["bias_grad"], what=name + " bias grad")


# ------------------------------------------------------------------ seeded cases vs the oracle

@pytest.mark.parametrize("D,R,in_f,out_f,anti", [
    (64, 2, 256, 192, True),      # vector path, two repeats
    (7, 5, 130, 67, True),        # odd sizes, scalar path, R = 4 + 1 passes
    (1, 1, 33, 1, False),         # single member, single output
    (16, 3, 64, 300, False),
])
def test_perturbed_linear_vs_oracle(base, D, R, in_f, out_f, anti):
    g = gen(100 + D)
    x = torch.randn(R * D, in_f, generator=g)
    W = torch.randn(out_f, in_f, generator=g) / in_f ** .5
    b = torch.randn(out_f, generator=g)
    E = 0.02 * torch.randn(D, out_f, in_f, generator=g)
    beta = 0.02 * torch.randn(D, out_f, generator=g)
    w = torch.rand(D, generator=g) * 2 - 1
    layer = base.PerturbedLinear(in_f, out_f, D, antithetic=anti).to(DEV)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(E), G(beta)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
        layer.perturbed_flag = False
        grad, bgrad = layer.update(G(w), l2=0.01)
    assert_close(y, O.perturbed_linear_forward(x, W, b, E, beta, D, anti), what="forward")
    # the ES signal is the member-to-member difference: check it on its own scale too
    base_y = torch.nn.functional.linear(x, W, b)
    assert_close(y.cpu() - base_y, O.perturbed_linear_forward(x, W, b, E, beta, D, anti) - base_y, tol=1e-3,
                 what="perturbation term")
    og, obg = O.perturbed_update(W, E, beta, w, 0, 0.01)
    assert_close(grad, og, what="grad")
    assert_close(bgrad, obg, what="bias grad")


@pytest.mark.parametrize("mode,in_sp,out_sp,repeats", [
    ("out", 0, 0, False), ("in", 0, 0, False), ("both", 0, 0, False),
    ("out", 0, 0.25, False), ("in", 0.1, 0, False), ("auto", 0.5, 0.5, False), ("in", 40, 0, True),
])
def test_permuted_linear_vs_oracle(base, mode, in_sp, out_sp, repeats):
    D, R, in_f, out_f = 48, 2, 200, 136
    g = gen(7)
    layer = base.PermutedLinear(in_f, out_f, D, antithetic=True, permutation=mode, in_sparsity=in_sp,
                                out_sparsity=out_sp, options={"allow_repeats": True} if repeats else {}).to(DEV)
    isp, osp = layer.in_sparsity, layer.out_sparsity
    x = torch.randn(R * D, in_f, generator=g)
    W = torch.randn(out_f, in_f, generator=g) / in_f ** .5
    b = torch.randn(out_f, generator=g)
    eps = 0.05 * torch.randn(osp, isp, generator=g)
    beta = 0.02 * torch.randn(D, out_f, generator=g)
    pin = pout = None
    if layer.permute_inputs:
        pin = torch.randint(in_f, (D, isp), generator=g).short() if repeats else perms(g, D, in_f, isp)
    if layer.permute_outputs:
        pout = perms(g, D, out_f)
    w = torch.randn(D, generator=g)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(eps), G(beta)
    layer.input_permutations, layer.output_permutations = G(pin), G(pout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
        layer.perturbed_flag = False
        grad, bgrad = layer.update(G(w), l1=0.001)
    assert_close(y, O.permuted_linear_forward(x, W, b, eps, beta, pin, pout, D, True), what="forward")
    og = O.permuted_linear_weight_grad(eps, w, pin, pout, in_f, out_f) + 0.001 * torch.sign(W)
    assert_close(grad, og, what="grad")
    assert_close(bgrad, w @ beta, what="bias grad")


@pytest.mark.parametrize("mode,in_sp,out_sp,stride,pad,k,R", [
    ("out", 0, 0.5, 1, 1, 3, 1), ("in", 0, 0, 1, 1, 3, 2), ("both", 0, 0, 2, 0, 3, 1),
    ("out", 0, 0, 1, 0, 1, 3), ("auto", 0.5, 0, 1, 2, 5, 1),
])
def test_permuted_conv_vs_oracle(base, mode, in_sp, out_sp, stride, pad, k, R):
    D, cin, cout, hw = 6, 10, 12, 13
    g = gen(11)
    layer = base.PermutedConv2d(cin, cout, k, D, stride=stride, padding=pad, antithetic=True, permutation=mode,
                                in_sparsity=in_sp, out_sparsity=out_sp).to(DEV)
    isp, osp = layer.in_sparsity, layer.out_sparsity
    x = torch.randn(R * D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g)
    eps = 0.05 * torch.randn(osp, isp, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g)
    pin = perms(g, D, cin, isp) if layer.permute_inputs else None
    pout = perms(g, D, cout) if layer.permute_outputs else None
    w = torch.randn(D, generator=g)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(eps), G(beta)
    layer.input_permutations, layer.output_permutations = G(pin), G(pout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
        layer.perturbed_flag = False
        y_off = layer.forward(G(x))
        grad, bgrad = layer.update(G(w))
    assert_close(y, O.permuted_conv2d_forward(x, W, b, eps, beta, pin, pout, D, stride, pad, 1, True), what="forward")
    assert_close(y_off, torch.nn.functional.conv2d(x, W, b, stride, pad), what="inference")
    assert_close(grad, O.permuted_conv2d_weight_grad(eps, w, pin, pout, cin, cout), what="grad")
    assert_close(bgrad, w @ beta, what="bias grad")


def test_permuted_conv_allow_repeats_uses_dense_noise(base):
    D, cin, cout, hw, k = 5, 6, 4, 7, 3
    g = gen(13)
    layer = base.PermutedConv2d(cin, cout, k, D, padding=1, permutation="in", in_sparsity=4,
                                options={"allow_repeats": True}).to(DEV)
    x = torch.randn(D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) * .2
    b = torch.randn(cout, generator=g)
    eps = 0.05 * torch.randn(cout, 4, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g)
    pin = torch.randint(cin, (D, 4), generator=g).short()
    pin[0, 1] = pin[0, 0]            # force a repeat
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.input_permutations = G(eps), G(beta), G(pin)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    assert_close(y, O.permuted_conv2d_forward(x, W, b, eps, beta, pin, None, D, 1, 1, 1, False), what="forward")


def test_perturbed_conv_vs_oracle(base):
    D, R, cin, cout, hw, k = 5, 3, 7, 70, 12, 3     # cout > 64 exercises the 128-wide tile
    g = gen(17)
    x = torch.randn(R * D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g)
    E = 0.05 * torch.randn(D, cout, cin, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g)
    layer = base.PerturbedConv2d(cin, cout, k, D, padding=1, antithetic=True).to(DEV)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(E), G(beta)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    assert_close(y, O.perturbed_conv2d_forward(x, W, b, E, beta, D, 1, 1, 1, True), what="forward")


@pytest.mark.parametrize("k", [1, 2, 5])
def test_sparse_perturbed_linear_vs_dense_reference_form(base, k):
    D, R, in_f, out_f = 12, 2, 96, 40
    g = gen(19 + k)
    x = torch.randn(R * D, in_f, generator=g)
    W = torch.randn(out_f, in_f, generator=g) / in_f ** .5
    b = torch.randn(out_f, generator=g)
    idx = torch.randint(in_f, (D, out_f, k), generator=g).int()
    val = 0.1 * torch.randn(D, out_f, k, generator=g)
    beta = 0.02 * torch.randn(D, out_f, generator=g)
    w = torch.randn(D, generator=g)
    layer = base.SparsePerturbedLinear(in_f, out_f, D, antithetic=True, k=k).to(DEV)
    set_params(layer, W, b)
    layer.weight_noise, layer.noise_indices, layer.bias_noise = G(val), G(idx), G(beta)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
        layer.perturbed_flag = False
        grad, bgrad = layer.update(G(w))
    assert layer.last_path == "3xtf32"           # base product on the tensor cores, k-entry gather in a second pass
    want = O.sparse_perturbed_linear_forward(x, W, b, idx, val, beta, D, True)
    assert_close(y, want, what="forward")
    layer.options = {"tc": "fp32"}
    with torch.no_grad():
        layer.perturbed_flag = True
        y32 = layer.forward(G(x))
        layer.perturbed_flag = False
    assert layer.last_path == "fp32"
    assert_close(y32, want, what="forward on CUDA cores")
    E = O.densify_sparse_noise(idx, val, in_f)
    assert_close(grad, O.perturbed_weight_grad(E, w), what="grad")
    assert_close(bgrad, w @ beta, what="bias grad")


# ------------------------------------------------------------------ benchmark configurations

def test_config1_permuted_linear_full_size(base):
    """PermutedLinear 256x256, 512 antithetic pairs, rank-normalised update."""
    D, R, n = 512, 2, 256
    g = gen(1001)
    x = torch.randn(R * D, n, generator=g)
    W = torch.randn(n, n, generator=g) / n ** .5
    eps = 0.02 * torch.randn(n, n, generator=g)
    beta = 0.02 * torch.randn(D, n, generator=g)
    pout = perms(g, D, n)
    u = O.centered_ranks(torch.randn(R * D, generator=g))
    w = u[:D] - u[D:]
    layer = base.PermutedLinear(n, n, D, antithetic=True).to(DEV)
    assert layer.permute_outputs and not layer.permute_inputs
    set_params(layer, W, torch.zeros(n))
    layer.weight_noise, layer.bias_noise, layer.output_permutations = G(eps), G(beta), G(pout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
        layer.perturbed_flag = False
        grad, bgrad = layer.update(G(w))
    assert_close(y, O.permuted_linear_forward(x, W, torch.zeros(n), eps, beta, None, pout, D, True), what="forward")
    assert_close(grad, O.permuted_linear_weight_grad(eps, w, None, pout, n, n), what="grad")
    assert_close(bgrad, w @ beta, what="bias grad")


def test_config2_perturbed_linear_full_size_properties(base):
    """PerturbedLinear 1024x1024 with 1024 dense noise matrices (4 GiB): checked through
    size-independent properties and an oracle comparison on a slice of members / columns."""
    D, R, n = 1024, 2, 1024
    torch.manual_seed(1002)
    layer = base.PerturbedLinear(n, n, D, antithetic=True).to(DEV)
    layer.set_seed(1234)
    layer.set_noise(0.02)
    E = layer.weight_noise
    assert tuple(E.shape) == (D, n, n)
    assert abs(E[:8].std().item() - 0.02) < 2e-4 and abs(E[:8].mean().item()) < 1e-4
    x = torch.randn(R * D, n, device=DEV)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(x)
        # antithetic symmetry: with the same input on both repeats, y+ + y- = 2 * (xW^T + b) exactly up to rounding
        xs = torch.cat([x[:D], x[:D]])
        ys = layer.forward(xs)
        layer.perturbed_flag = False
        base_y = layer.forward(x[:D])
    assert_close((ys[:D] + ys[D:]) / 2, base_y.cpu(), what="antithetic symmetry")
    # oracle on a slice of members
    sel = [0, 1, 511, 1023]
    Ws, bs = layer.weight.detach().cpu(), layer.bias.detach().cpu()
    for d in sel:
        Ed, bd = E[d].cpu(), layer.bias_noise[d].cpu()
        for r, s in ((0, 1.0), (1, -1.0)):
            xr = x[r * D + d].cpu()
            want = Ws @ xr + bs + s * (Ed @ xr + bd)
            assert_close(y[r * D + d], want, what="member %d repeat %d" % (d, r))
    # update: one-hot weights return that member's noise bit-exactly; random weights vs oracle on columns
    w = torch.zeros(D, device=DEV)
    w[777] = 1.0
    with torch.no_grad():
        g1 = layer.weight_grad(w)
    assert torch.equal(g1, E[777])
    w = torch.rand(D, device=DEV) * 2 - 1
    with torch.no_grad():
        g2 = layer.weight_grad(w)
    cols = E.view(D, -1)[:, 12345:12345 + 4096].cpu()
    assert_close(g2.view(-1)[12345:12345 + 4096], w.cpu() @ cols, what="update slice")
    # linearity in the weights
    with torch.no_grad():
        g3 = layer.weight_grad(2 * w)
    assert_close(g3, 2 * g2.cpu(), tol=1e-6, what="linearity")


def test_config3_permuted_conv_full_size(base):
    """PermutedConv2d 64->64 3x3 pad 1 on 32x32, population 1024, out_sparsity 0.5."""
    D, c, hw = 1024, 64, 32
    g = gen(1003)
    layer = base.PermutedConv2d(c, c, 3, D, padding=1, out_sparsity=.5).to(DEV)
    assert layer.out_sparsity == 32 and layer.permute_outputs and not layer.permute_inputs
    x = torch.randn(D, c, hw, hw, generator=g)
    W = torch.randn(c, c, 3, 3, generator=g) * (2 / 576) ** .5
    b = torch.zeros(c)
    eps = 0.02 * 2 ** .5 * torch.randn(32, c, 3, 3, generator=g)
    beta = 0.02 * torch.randn(D, c, generator=g)
    pout = perms(g, D, c)
    w = torch.randn(D, generator=g)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.output_permutations = G(eps), G(beta), G(pout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
        layer.perturbed_flag = False
        grad, bgrad = layer.update(G(w))
    want = O.permuted_conv2d_forward(x, W, b, eps, beta, None, pout, D, 1, 1, 1, False)
    assert_close(y, want, what="forward")
    basey = torch.nn.functional.conv2d(x[:16], W, b, 1, 1)
    assert_close(y[:16].cpu() - basey, want[:16] - basey, tol=1e-3, what="perturbation term")
    assert_close(grad, O.permuted_conv2d_weight_grad(eps, w, None, pout, c, c), what="grad")


# ------------------------------------------------------------------ edge cases and errors

def test_edge_cases_and_errors(base):
    layer = base.PermutedLinear(8, 6, 4).to(DEV)
    layer.set_noise(0.1)
    assert layer.weight_noise.shape == (6, 8)
    layer.perturbed_flag = True
    with torch.no_grad():
        assert layer.forward(torch.zeros(0, 8, device=DEV)).shape == (0, 6)       # empty batch
        with pytest.raises(RuntimeError):
            layer.forward(torch.zeros(6, 8, device=DEV))                             # not a multiple of directions
        with pytest.raises(RuntimeError):
            layer.forward(torch.zeros(4, 8))                                         # CPU tensor: no fallback
        with pytest.raises(NotImplementedError):
            layer.forward(torch.zeros(4, 8, device=DEV, dtype=torch.float16))
        with pytest.raises(RuntimeError):
            layer.update(torch.zeros(3, device=DEV))
    # permutations drawn on the device are permutations
    big = base.PermutedLinear(300, 200, 64, permutation="both", in_sparsity=37).to(DEV)
    big.set_seed(5)
    big.set_noise(0.02)
    po = big.output_permutations.cpu().long()
    assert po.shape == (64, 200) and torch.equal(po.sort(dim=1).values, torch.arange(200).expand(64, 200))
    pi = big.input_permutations.cpu().long()
    assert pi.shape == (64, 37) and all(len(set(r.tolist())) == 37 for r in pi) and pi.max() < 300 and pi.min() >= 0
    assert not torch.equal(po[0], po[1])
    again = base.PermutedLinear(300, 200, 64, permutation="both", in_sparsity=37).to(DEV)
    again.set_seed(5)
    again.set_noise(0.02)
    assert torch.equal(again.output_permutations, big.output_permutations)           # same seed, same draw
    assert torch.equal(again.weight_noise, big.weight_noise)
    rescale = (200 * 300 / 200 / 37) ** .5
    assert abs(big.weight_noise.std().item() / (0.02 * rescale) - 1) < 0.05


def test_population_model_end_to_end(base):
    D = 8
    net = torch.nn.Sequential(base.PermutedConv2d(1, 4, 3, D), torch.nn.ReLU(), torch.nn.Flatten(),
                              base.PermutedLinear(4 * 6 * 6, 5, D)).to(DEV)
    pm = base.PerturbedModel(net, D)
    pm.set_noise_scale(0.05)
    pm.set_seed(3)
    pm.allocate_memory()
    pm.set_noise()
    x = torch.rand(2 * D, 1, 8, 8, device=DEV)
    with torch.no_grad():
        out = pm.forward(x)
        plain = net(x)
        assert out.shape == (2 * D, 5) and not torch.equal(out, plain)
        pm.update(torch.randn(D, device=DEV))
    assert all(p.grad is not None for p in net.parameters())
    pm.free_memory()
    assert net[0].weight_noise is None and net[3].input_permutations is None


@pytest.mark.parametrize("cin,cout,out_sp,hw,k,pad,R,anti,bias", [
    (1, 32, 0, 28, 3, 0, 3, False, True),      # first layer of the small CNN
    (3, 40, 0.5, 15, 3, 1, 4, True, True),     # odd output size (floor pooling), sparsity, antithetic halves
    (2, 8, 0, 9, 2, 0, 1, True, False),
    # 16-channel multiples take the table form: odd map width (no paired loads), sparsity, antithetic halves, no bias
    (3, 48, 0.5, 15, 3, 1, 4, True, True), (2, 16, 0.25, 11, 2, 0, 2, True, False),
])
def test_shared_input_conv_relu_pool(base, cin, cout, out_sp, hw, k, pad, R, anti, bias):
    """options shared_input + fuse: every member sees the same images; result equals the oracle's layer on the
    expanded batch followed by ReLU and MaxPool2d(2), returned as a channels-last tensor."""
    D = 12
    g = gen(31 + cout)
    layer = base.PermutedConv2d(cin, cout, k, D, padding=pad, bias=bias, antithetic=anti, permutation="out",
                                out_sparsity=out_sp, options={"shared_input": True, "fuse": "relu_maxpool2"}).to(DEV)
    osp = layer.out_sparsity
    x = torch.rand(R, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g) * .1 if bias else None
    eps = 0.05 * torch.randn(osp, cin, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g) if bias else None
    pout = perms(g, D, cout)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.output_permutations = G(eps), (G(beta) if bias else None), G(pout)
    xb = x.unsqueeze(1).expand(R, D, cin, hw, hw).reshape(R * D, cin, hw, hw).contiguous()
    want = O.permuted_conv2d_forward(xb, W, b if bias else torch.zeros(cout), eps,
                                     beta if bias else torch.zeros(D, cout), None, pout, D, 1, pad, 1, anti)
    want = torch.nn.functional.max_pool2d(torch.relu(want), 2)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
        layer.perturbed_flag = False
        y_off = layer.forward(G(x))
    assert y.shape == want.shape and y.is_contiguous(memory_format=torch.channels_last)
    assert_close(y, want, what="fused forward")
    plain = torch.nn.functional.conv2d(x, W, b, 1, pad)
    assert_close(y_off, torch.nn.functional.max_pool2d(torch.relu(plain), 2), what="inference")
    # reduced-precision stores for a tensor-core consumer: the same values rounded once
    for out, step in (("tf32", 2.0 ** -11), ("bf16", 2.0 ** -8)):
        layer.options = dict(layer.options, out_dtype=out)
        with torch.no_grad():
            layer.perturbed_flag = True
            yr = layer.forward(G(x))
            layer.perturbed_flag = False
        assert yr.dtype == (torch.bfloat16 if out == "bf16" else torch.float32)
        assert torch.all((yr.float() - y).abs() <= step * y.abs() + 1e-30)
    # pair layout: images 2q and 2q+1 interleaved by pixel, presented as R*D/2 images of 2*C channels
    layer.options = dict(layer.options, out_dtype="bf16x2")
    with torch.no_grad():
        layer.perturbed_flag = True
        yp = layer.forward(G(x))
        layer.perturbed_flag = False
    Hp, Wp = y.shape[2:]
    assert yp.dtype == torch.bfloat16 and tuple(yp.shape) == (R * D // 2, 2 * cout, Hp, Wp)
    pairs = yp.permute(0, 2, 3, 1).reshape(R * D // 2, Hp, Wp, 2, cout).permute(0, 3, 4, 1, 2).reshape(R * D, cout, Hp, Wp)
    assert torch.all((pairs.float() - y).abs() <= 2.0 ** -8 * y.abs() + 1e-30)


def test_fuse_option_falls_back_to_separate_kernels(base):
    """fuse without a fused kernel for the case (input permutations): same numbers through conv + torch ops."""
    D, R, cin, cout, hw = 6, 2, 10, 12, 11
    g = gen(41)
    layer = base.PermutedConv2d(cin, cout, 3, D, permutation="in", options={"fuse": "relu_maxpool2"}).to(DEV)
    x = torch.randn(R * D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, 3, 3, generator=g) * .1
    b = torch.randn(cout, generator=g) * .1
    eps = 0.05 * torch.randn(cout, cin, 3, 3, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g)
    pin = perms(g, D, cin)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.input_permutations = G(eps), G(beta), G(pin)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    want = O.permuted_conv2d_forward(x, W, b, eps, beta, pin, None, D, 1, 0, 1, False)
    assert_close(y, torch.nn.functional.max_pool2d(torch.relu(want), 2), what="forward")


def test_fused_layer_edge_cases(base):
    """Empty batches pass through the fused layers; an unknown fuse option is refused."""
    D = 4
    shared = base.PermutedConv2d(1, 8, 3, D, permutation="out", options={"shared_input": True, "fuse": "relu_maxpool2"}).to(DEV)
    shared.allocate_memory()
    shared.set_seed(3)
    shared.set_noise(0.02)
    shared.perturbed_flag = True
    with torch.no_grad():
        y = shared.forward(torch.zeros(0, 1, 10, 10, device=DEV))
    assert tuple(y.shape) == (0, 8, 4, 4)
    tc = base.PermutedConv2d(32, 16, 3, D, permutation="out", options={"tc": "tf32", "fuse": "relu_maxpool2"}).to(DEV)
    tc.allocate_memory()
    tc.set_seed(4)
    tc.set_noise(0.02)
    tc.perturbed_flag = True
    with torch.no_grad():
        y = tc.forward(torch.zeros(0, 32, 13, 13, device=DEV))
    assert tuple(y.shape) == (0, 16, 5, 5)
    bad = base.PermutedConv2d(1, 8, 3, D, options={"fuse": "relu"}).to(DEV)
    with pytest.raises(NotImplementedError):
        bad.forward(torch.zeros(D, 1, 10, 10, device=DEV))


def test_weight_gradient_in_column_blocks_and_overlapped_update(base):
    """The block-by-block form of the dense update (the one that feeds an all-reduce block by block) against the
    oracle and against the one-shot update; with a single process the overlapped update is just the blocks."""
    from nesgpu_b200 import dist as ndist
    D, in_f, out_f = 40, 96, 50
    g = gen(77)
    layer = base.PerturbedLinear(in_f, out_f, D).to(DEV)
    E = 0.1 * torch.randn(D, out_f, in_f, generator=g)
    beta = 0.1 * torch.randn(D, out_f, generator=g)
    w = torch.randn(D, generator=g)
    layer.weight_noise, layer.bias_noise = G(E), G(beta)
    want = O.perturbed_weight_grad(E, w).flatten()
    n = out_f * in_f
    for lo, hi in [(0, n), (0, 1024), (1024, 4096), (4096, n), (3, 1001)]:
        out = torch.empty(hi - lo, device=DEV)
        layer.weight_grad_columns(G(w), lo, hi, out)
        assert_close(out, want[lo:hi], what="columns %d:%d" % (lo, hi))
    with torch.no_grad():
        bucket = ndist.overlapped_dense_update(layer, G(w), blocks=3, l2=0.01)
    og, obg = O.perturbed_update(layer.weight.detach().cpu(), E, beta, w, 0, 0.01)
    assert_close(layer.weight.grad, og, what="overlapped grad")
    assert_close(layer.bias.grad, obg, what="overlapped bias grad")
    assert layer.weight.grad.data_ptr() == bucket.views()[0].data_ptr()
    # the next plain update starts from an empty .grad and lands in the same bucket slice
    layer.weight.grad = layer.bias.grad = None
    with torch.no_grad():
        grad, bgrad = layer.update(G(w), l2=0.01)
    assert grad.data_ptr() == bucket.views()[0].data_ptr() and bgrad.data_ptr() == bucket.views()[1].data_ptr()
    assert_close(grad, og, what="bucket-resident grad")


def test_device_normal_fill_distribution_and_layout_independence():
    """The Philox / Box-Muller fill: moments and tails of 16 M samples, and the value at index i depends only on
    (seed, offset + i / 4) -- not on the launch shape, the size or the alignment of the tensor."""
    from nesgpu_b200 import _cabi as C
    n = 1 << 24
    t = torch.empty(n, device=DEV)
    C.call("nes_fill_normal", C.ptr(t), n, 1.5, 2.0, 1234, 0, C.stream())
    z = (t.double() - 1.5) / 2.0
    assert abs(z.mean().item()) < 1.5e-3 and abs(z.std().item() - 1) < 1e-3
    assert abs((z ** 3).mean().item()) < 5e-3 and abs((z ** 4).mean().item() - 3) < 2e-2
    assert abs((z.abs() > 3).double().mean().item() / 0.0026998 - 1) < 0.05
    assert 4.5 < z.abs().max().item() < 5.8                       # 24-bit uniforms cap the radius at 5.77
    # same counters, other shapes: a shorter tensor, and one that starts 4 bytes into an allocation (scalar stores)
    short = torch.empty(1001, device=DEV)
    C.call("nes_fill_normal", C.ptr(short), 1001, 1.5, 2.0, 1234, 0, C.stream())
    assert torch.equal(short, t[:1001])
    raw = torch.empty(4097, device=DEV)
    view = raw[1:]
    C.call("nes_fill_normal", C.ptr(view), 4096, 1.5, 2.0, 1234, 0, C.stream())
    assert torch.equal(view, t[:4096])
    later = torch.empty(4096, device=DEV)
    C.call("nes_fill_normal", C.ptr(later), 4096, 1.5, 2.0, 1234, 1024, C.stream())
    assert torch.equal(later, t[4096:8192])
