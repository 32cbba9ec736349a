"""GPU parity of the sign-flip (Synthetic) layers and PerturbedAffine against the golden vectors produced by the
reference and against the oracle on seeded inputs."""
import pytest
import torch

from gpu_util import DEV, G, T, assert_close, set_params
from oracle import perturbed_ref as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def base():
    from nesgpu_b200 import base as b
    return b


def test_golden_synthetic_linear(base, perturbed_golden):
    for name in perturbed_golden.names("SyntheticLinear"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        layer = base.SyntheticLinear(m["in_f"], m["out_f"], m["D"], antithetic=m["antithetic"], flip=m["flip"]).to(DEV)
        assert (layer.flip_inputs, layer.flip_outputs) == (m["flip_inputs"], m["flip_outputs"])
        set_params(layer, c["weight"], c["bias"])
        layer.weight_noise, layer.bias_noise = G(c["weight_noise"]), G(c["bias_noise"])
        layer.input_flips, layer.output_flips = G(c.get("fin")), G(c.get("fout"))
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(G(c["x"]))
            layer.perturbed_flag = False
            grad, bgrad = layer.update(G(c["w"]))
        assert_close(y, c["y"], what=name + " forward")
        want = c["grad"] if "grad" in c else O.synthetic_weight_grad(T(c["weight_noise"]), T(c["w"]), T(c.get("fin")), T(c.get("fout")))
        assert_close(grad, want, what=name + " grad")
        assert_close(bgrad, T(c["w"]) @ T(c["bias_noise"]), what=name + " bias grad")


def test_golden_synthetic_conv(base, perturbed_golden):
    for name in perturbed_golden.names("SyntheticConv2d"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        layer = base.SyntheticConv2d(m["cin"], m["cout"], m["k"], m["D"], stride=m["stride"], padding=m["padding"],
                                     antithetic=m["antithetic"], flip=m["flip"]).to(DEV)
        set_params(layer, c["weight"], c["bias"])
        layer.weight_noise, layer.bias_noise = G(c["weight_noise"]), G(c["bias_noise"])
        layer.input_flips, layer.output_flips = G(c.get("fin")), G(c.get("fout"))
        with torch.no_grad():
            layer.perturbed_flag = True
            y = layer.forward(G(c["x"]))
            layer.perturbed_flag = False
            grad, _ = layer.update(G(c["w"]))
        assert_close(y, c["y"], what=name + " forward")
        want = c["grad"] if "grad" in c else O.synthetic_weight_grad(T(c["weight_noise"]), T(c["w"]), T(c.get("fin")), T(c.get("fout")))
        assert_close(grad, want, what=name + " grad")


@pytest.mark.parametrize("flip", ["in", "out", "both"])
def test_synthetic_vs_oracle_midsize(base, flip):
    D, R, in_f, out_f = 40, 3, 130, 72
    g = torch.Generator().manual_seed(3)
    layer = base.SyntheticLinear(in_f, out_f, D, antithetic=True, flip=flip).to(DEV)
    x = torch.randn(R * D, in_f, generator=g)
    W = torch.randn(out_f, in_f, generator=g) / in_f ** .5
    b = torch.randn(out_f, generator=g)
    eps = 0.05 * torch.randn(out_f, in_f, generator=g)
    beta = 0.02 * torch.randn(D, out_f, generator=g)
    fi = (2 * torch.randint(2, (D, in_f), generator=g) - 1).to(torch.int8) if layer.flip_inputs else None
    fo = (2 * torch.randint(2, (D, out_f), generator=g) - 1).to(torch.int8) if layer.flip_outputs else None
    w = torch.randn(D, generator=g)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.input_flips, layer.output_flips = G(eps), G(beta), G(fi), G(fo)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
        layer.perturbed_flag = False
        grad, _ = layer.update(G(w), l2=0.1)
    assert_close(y, O.synthetic_linear_forward(x, W, b, eps, beta, fi, fo, D, True), what="forward")
    assert_close(grad, O.synthetic_weight_grad(eps, w, fi, fo) + 0.1 * W, what="grad")
    # conv with repeats > 1 (the reference's own broadcast only works for R == 1)
    conv = base.SyntheticConv2d(6, 10, 3, D, padding=1, antithetic=True, flip=flip).to(DEV)
    xc = torch.randn(2 * D, 6, 9, 9, generator=g)
    Wc = torch.randn(10, 6, 3, 3, generator=g) * .2
    bc = torch.randn(10, generator=g)
    ec = 0.05 * torch.randn(10, 6, 3, 3, generator=g)
    bnc = 0.02 * torch.randn(D, 10, generator=g)
    fic = (2 * torch.randint(2, (D, 6), generator=g) - 1).to(torch.int8) if conv.flip_inputs else None
    foc = (2 * torch.randint(2, (D, 10), generator=g) - 1).to(torch.int8) if conv.flip_outputs else None
    set_params(conv, Wc, bc)
    conv.weight_noise, conv.bias_noise, conv.input_flips, conv.output_flips = G(ec), G(bnc), G(fic), G(foc)
    with torch.no_grad():
        conv.perturbed_flag = True
        yc = conv.forward(G(xc))
    assert_close(yc, O.synthetic_conv2d_forward(xc, Wc, bc, ec, bnc, fic, foc, D, 1, 1, 1, True), what="conv forward")


def test_synthetic_set_noise_and_affine(base, perturbed_golden):
    layer = base.SyntheticLinear(64, 48, 32, flip="both").to(DEV)
    layer.set_seed(4)
    layer.set_noise(0.05)
    assert layer.input_flips.shape == (32, 64) and layer.output_flips.dtype == torch.int8
    assert set(layer.input_flips.unique().tolist()) == {-1, 1}
    assert abs(layer.output_flips.float().mean().item()) < 0.15
    assert abs(layer.weight_noise.std().item() / 0.05 - 1) < 0.1
    m, c = perturbed_golden.meta["affine"], perturbed_golden.case("affine")
    aff = base.PerturbedAffine(tuple(m["shape"]), m["D"]).to(DEV)
    set_params(aff, c["weight"], c["bias"])
    aff.weight_noise, aff.bias_noise = G(c["weight_noise"]), G(c["bias_noise"])
    with torch.no_grad():
        aff.perturbed_flag = True
        y = aff.forward(G(c["x"]))
        aff.perturbed_flag = False
        grad, bgrad = aff.update(G(c["w"]))
    assert_close(y, c["y"], what="affine forward")
    # the stored tensors are W + noise; the kernel subtracts W row by row, as the reference does, so the fp32 bar holds
    assert_close(grad, c["grad"], what="affine grad")
    assert_close(bgrad, c["bias_grad"], what="affine bias grad")
    aff.set_seed(1)
    aff.set_noise(0.1)
    assert aff.weight_noise.shape == (m["D"],) + tuple(m["shape"])


@pytest.mark.parametrize("flip", ["in", "out", "both"])
@pytest.mark.parametrize("tc,tol", [("3xtf32", 1e-4), ("tf32", 2e-2), ("fp32", 1e-4)])
def test_synthetic_linear_tensor_core_products(base, flip, tc, tol):
    """Row lengths that are multiples of 4 take the two tcgen05 products (3xTF32 by default: the fp32 bar; plain
    TF32 is the stated reduced-precision mode); the perturbation term is checked on its own as well."""
    D, R, in_f, out_f = 24, 2, 256, 136
    g = torch.Generator().manual_seed(13)
    layer = base.SyntheticLinear(in_f, out_f, D, antithetic=True, flip=flip, options={"tc": tc}).to(DEV)
    x = torch.randn(R * D, in_f, generator=g)
    W = torch.randn(out_f, in_f, generator=g) / in_f ** .5
    b = torch.randn(out_f, generator=g)
    eps = 0.05 * torch.randn(out_f, in_f, generator=g)
    beta = 0.02 * torch.randn(D, out_f, generator=g)
    fin = (2 * torch.randint(2, (D, in_f), generator=g) - 1).to(torch.int8) if layer.flip_inputs else None
    fout = (2 * torch.randint(2, (D, out_f), generator=g) - 1).to(torch.int8) if layer.flip_outputs else None
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.input_flips, layer.output_flips = G(eps), G(beta), G(fin), G(fout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    assert layer.last_path == tc
    want = O.synthetic_linear_forward(x, W, b, eps, beta, fin, fout, D, True)
    assert_close(y, want, tol=tol, what="forward")
    base_only = x @ W.t() + b
    assert_close(y.cpu() - base_only, want - base_only, tol=10 * tol, what="perturbation term")
