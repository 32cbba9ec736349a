"""The ES step on the small CNN of the last benchmark configuration (reduced population), against the
CPU oracle evaluated layer by layer on the same injected noise."""
import pytest
import torch
import torch.nn.functional as F

from gpu_util import DEV, assert_close, rel_err
from oracle import perturbed_ref as O

pytestmark = pytest.mark.gpu


def build(base, D):
    return torch.nn.Sequential(
        base.PermutedConv2d(1, 32, 3, D), torch.nn.ReLU(), torch.nn.MaxPool2d(2),
        base.PermutedConv2d(32, 64, 3, D), torch.nn.ReLU(), torch.nn.MaxPool2d(2), torch.nn.Flatten(),
        base.PermutedLinear(1600, 128, D), torch.nn.ReLU(), base.PermutedLinear(128, 10, D)).to(DEV)


def oracle_forward(layers, x, D):
    c = lambda t: None if t is None else t.detach().cpu()
    for layer in layers:
        name = type(layer).__name__
        if name == "PermutedConv2d":
            x = O.permuted_conv2d_forward(x, c(layer.weight), c(layer.bias), c(layer.weight_noise), c(layer.bias_noise),
                                          c(layer.input_permutations), c(layer.output_permutations), D, 1, 0, 1, False)
        elif name == "PermutedLinear":
            x = O.permuted_linear_forward(x, c(layer.weight), c(layer.bias), c(layer.weight_noise), c(layer.bias_noise),
                                          c(layer.input_permutations), c(layer.output_permutations), D, False)
        else:
            x = layer(x)
    return x


def test_es_step_small_population():
    from nesgpu_b200 import base, es
    D, R = 6, 5
    torch.manual_seed(0)
    net = build(base, D)
    pm = base.PerturbedModel(net, D)
    modes = [(l.permute_inputs, l.permute_outputs) for l in pm.perturbed_layers]
    assert modes == [(False, True), (False, True), (True, False), (True, False)]     # auto: out, out, in, in
    pm.set_noise_scale(0.02)
    pm.set_seed(11)
    images = torch.rand(R, 1, 28, 28, device=DEV)
    labels = torch.randint(10, (R,), device=DEV)
    fitness, _ = es.es_step(pm, images, labels, D, chunk=2)
    # oracle: same noise, whole batch at once
    xb = images.cpu().unsqueeze(1).expand(R, D, 1, 28, 28).reshape(R * D, 1, 28, 28)
    logits = oracle_forward(list(net), xb, D)
    ce = F.cross_entropy(logits, labels.cpu().repeat_interleave(D), reduction="none").view(R, D)
    want_fit = -ce.mean(dim=0)
    assert_close(fitness, want_fit, tol=1e-4, what="fitness")
    assert torch.equal(es.centered_ranks(fitness).cpu(), O.centered_ranks(want_fit))
    # .grad is a descent gradient: the reference's trainer weights members by (loss - mean) / noise_scale
    # (mnisttest.py:141-146); with rank-normalised negative loss that is -ranks / noise_scale
    w = -O.centered_ranks(want_fit) / 0.02
    assert torch.allclose(es.update_weights(fitness, 0.02).cpu(), w, rtol=1e-6, atol=0)
    c = lambda t: None if t is None else t.detach().cpu()
    for layer in pm.perturbed_layers:
        if type(layer).__name__ == "PermutedConv2d":
            g = O.permuted_conv2d_weight_grad(c(layer.weight_noise), w, c(layer.input_permutations),
                                              c(layer.output_permutations), layer.in_channels, layer.out_channels)
        else:
            g = O.permuted_linear_weight_grad(c(layer.weight_noise), w, c(layer.input_permutations),
                                              c(layer.output_permutations), layer.in_features, layer.out_features)
        assert_close(layer.weight.grad, g, tol=1e-4, what=type(layer).__name__ + " grad")
        assert_close(layer.bias.grad, w @ c(layer.bias_noise), tol=1e-4, what="bias grad")


def test_es_step_tensor_core_conv_close_to_fp32():
    """conv2 (32 -> 64 channels) on the TF32 tensor-core path: fitness within the stated reduced-precision bar."""
    from nesgpu_b200 import base, es
    D, R = 8, 4
    torch.manual_seed(1)
    net = build(base, D)
    pm = base.PerturbedModel(net, D)
    pm.set_noise_scale(0.02)
    pm.set_seed(5)
    pm.set_noise()
    images = torch.rand(R, 1, 28, 28, device=DEV)
    labels = torch.randint(10, (R,), device=DEV)
    f32 = es.population_fitness(pm, images, labels, D, chunk=4)
    net[3].options = {"tc": "tf32"}
    tf32 = es.population_fitness(pm, images, labels, D, chunk=4)
    assert rel_err(tf32, f32.cpu()) <= 2e-2
    assert not torch.equal(tf32, f32)


def build_fused(base, D, tc):
    """tc: None (exact fp32 kernels), "tf32" or "bf16" (the stated reduced-precision modes, all layers)."""
    pair = tc == "bf16x2"                     # bf16 with two images per tensor-core instruction in layer 2
    if pair:
        tc = "bf16"
    o1 = {"shared_input": True, "fuse": "relu_maxpool2", "out_dtype": "bf16x2" if pair else (tc or "fp32")}
    o2 = {"fuse": "relu_maxpool2"}
    lin = {}
    if tc == "bf16x3":                        # the fp32 bar on the tensor cores: split-bf16 layer 2, default linear layers
        o2["tc"] = tc
    elif tc:
        o2["tc"] = tc
        lin = {"tc": tc}
    if pair:
        o2["in_layout"] = "bf16x2"
    return torch.nn.Sequential(
        base.PermutedConv2d(1, 32, 3, D, options=o1),
        base.PermutedConv2d(32, 64, 3, D, options=o2), torch.nn.Flatten(),
        base.PermutedLinear(1600, 128, D, options=lin), torch.nn.ReLU(), base.PermutedLinear(128, 10, D, options=lin)).to(DEV)


@pytest.mark.parametrize("tc,tol", [(None, 1e-4), ("bf16x3", 1e-4), ("tf32", 2e-2), ("bf16", 2e-2), ("bf16x2", 2e-2)])
def test_es_step_fused_layers_match_the_module_by_module_network(tc, tol):
    """Same weights, noise and permutations in both networks: the fused Conv-ReLU-Pool layers (layer 1 fed with the
    shared minibatch) give the fitness of the Conv / ReLU / MaxPool2d network; exact-fp32 kernels hold 1e-4, the TF32
    mode its stated 2e-2."""
    from nesgpu_b200 import base, es
    D, R = 24, 6
    torch.manual_seed(2)
    plain = build(base, D)
    fused = build_fused(base, D, tc)
    pm_plain, pm_fused = base.PerturbedModel(plain, D), base.PerturbedModel(fused, D)
    pm_plain.set_noise_scale(0.02)
    pm_plain.set_seed(7)
    pm_plain.set_noise()
    pm_fused.set_noise_scale(0.02)
    pm_fused.set_seed(8)
    pm_fused.set_noise()
    for a, b in zip(pm_plain.perturbed_layers, pm_fused.perturbed_layers):
        with torch.no_grad():
            b.weight.copy_(a.weight)
            b.bias.copy_(a.bias)
        b.weight_noise, b.bias_noise = a.weight_noise, a.bias_noise
        b.input_permutations, b.output_permutations = a.input_permutations, a.output_permutations
    assert es.takes_shared_input(pm_fused) and not es.takes_shared_input(pm_plain)
    images = torch.rand(R, 1, 28, 28, device=DEV)
    labels = torch.randint(10, (R,), device=DEV)
    want = es.population_fitness(pm_plain, images, labels, D, chunk=4)
    got = es.population_fitness(pm_fused, images, labels, D, chunk=4)
    assert rel_err(got, want.cpu()) <= tol
    # inference (perturbed flag off): both networks are the plain CNN
    with torch.no_grad():
        assert_close(fused(images), plain(images).cpu(), tol=1e-4, what="inference")


def test_population_fitness_on_two_streams_equals_one_stream():
    from nesgpu_b200 import base, es
    D, R = 16, 12
    torch.manual_seed(3)
    net = build_fused(base, D, "bf16x2")
    pm = base.PerturbedModel(net, D)
    pm.set_noise_scale(0.02)
    pm.set_seed(21)
    pm.set_noise()
    images = torch.rand(R, 1, 28, 28, device=DEV)
    labels = torch.randint(10, (R,), device=DEV)
    one = es.population_fitness(pm, images, labels, D, chunk=3, streams=1)
    two = es.population_fitness(pm, images, labels, D, chunk=3, streams=2)
    three = es.population_fitness(pm, images, labels, D, chunk=3, streams=3)
    torch.cuda.synchronize()
    assert rel_err(two, one.cpu()) <= 1e-6 and rel_err(three, one.cpu()) <= 1e-6


def test_es_steps_followed_by_sgd_lower_the_loss():
    """.grad left by es_step is a descent direction: a few steps of plain SGD (minimising, as the reference's trainer
    uses, mnisttest.py:108,152) must lower the mean cross-entropy of the unperturbed network."""
    from nesgpu_b200 import base, es
    import random
    D, R = 256, 64
    torch.manual_seed(4)
    random.seed(4)
    net = torch.nn.Sequential(base.PermutedLinear(32, 64, D), torch.nn.ReLU(), base.PermutedLinear(64, 10, D)).to(DEV)
    pm = base.PerturbedModel(net, D)
    pm.set_noise_scale(0.05)
    x = torch.randn(R, 32, device=DEV)
    labels = torch.randint(10, (R,), device=DEV)
    opt = torch.optim.SGD(net.parameters(), lr=0.02)
    with torch.no_grad():
        before = F.cross_entropy(net(x), labels).item()
    for _ in range(10):
        es.es_step(pm, x, labels, D)
        opt.step()
        opt.zero_grad()
    with torch.no_grad():
        after = F.cross_entropy(net(x), labels).item()
    assert after < before - 0.05, (before, after)


def test_member_offset_gives_each_rank_its_slice_of_the_population():
    """Two "ranks" with the same seeds and member offsets 0 and 4 draw exactly the members 0-3 and 4-7 of an
    8-member layer (per-member tensors); the noise that all members share is identical everywhere."""
    from nesgpu_b200 import base
    whole = base.PermutedLinear(64, 48, 8, permutation="both").to(DEV)
    whole.set_seed(77)
    whole.set_noise(0.1)
    dense = base.PerturbedLinear(16, 8, 8).to(DEV)
    dense.set_seed(78)
    dense.set_noise(0.1)
    for lo in (0, 4):
        part = base.PermutedLinear(64, 48, 4, permutation="both").to(DEV)
        part.set_seed(77)
        part.set_member_offset(lo)
        part.set_noise(0.1)
        assert torch.equal(part.weight_noise, whole.weight_noise)
        assert torch.equal(part.bias_noise, whole.bias_noise[lo:lo + 4])
        assert torch.equal(part.input_permutations, whole.input_permutations[lo:lo + 4])
        assert torch.equal(part.output_permutations, whole.output_permutations[lo:lo + 4])
        dpart = base.PerturbedLinear(16, 8, 4).to(DEV)
        dpart.set_seed(78)
        dpart.set_member_offset(lo)
        dpart.set_noise(0.1)
        assert torch.equal(dpart.weight_noise, dense.weight_noise[lo:lo + 4])
        assert torch.equal(dpart.bias_noise, dense.bias_noise[lo:lo + 4])
    # rows that are not whole generator groups: the slices are not reproduced, but ranks never share draws
    odd_a, odd_b = base.PerturbedLinear(3, 3, 4).to(DEV), base.PerturbedLinear(3, 3, 4).to(DEV)
    for layer, lo in ((odd_a, 0), (odd_b, 4)):
        layer.set_seed(5)
        layer.set_member_offset(lo)
        layer.set_noise(0.1)
    assert not torch.isin(odd_a.weight_noise.flatten(), odd_b.weight_noise.flatten()).any()
