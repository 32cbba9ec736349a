"""GPU parity of the bit-packed ops (through nesgpu_b200.boolean_operations -> ctypes -> C ABI):
bit-exact against the numpy oracle and the golden vectors built from the reference's naive
formulas; the fp16 weighted sum within one fp16 rounding step."""
import numpy as np
import pytest
import torch

from gpu_util import DEV, G
from oracle import binary_ref as B

pytestmark = pytest.mark.gpu

DT = {32: torch.int32, 64: torch.int64}


@pytest.fixture(scope="module")
def ops():
    import nesgpu_b200.boolean_operations as bo
    return bo


def npy(t):
    return t.detach().cpu().numpy()


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("rows,cols", [(7, 150), (1, 1), (33, 64), (5, 1024), (3, 65)])
def test_pack_unpack(ops, bits, rows, cols):
    rng = np.random.default_rng(rows * 1000 + cols)
    b = rng.integers(0, 2, (rows, cols)).astype(bool)
    w = ops.pack(G(b), DT[bits])
    np.testing.assert_array_equal(npy(w), B.pack(b, bits))
    np.testing.assert_array_equal(npy(ops.unpack(w)), B.unpack(B.pack(b, bits), bits))
    by = rng.integers(0, 256, (rows, cols)).astype(np.uint8)
    np.testing.assert_array_equal(npy(ops.int8pack(G(by), DT[bits])), B.int8pack(by, bits))
    np.testing.assert_array_equal(npy(ops.pack8(G(b))), B.pack8(b))
    np.testing.assert_array_equal(npy(ops.unpack(ops.pack8(G(b))))[:, :cols], b)


@pytest.mark.parametrize("bits", [32, 64])
def test_golden_conv_act_pool(ops, binary_golden, bits):
    for name in binary_golden.names():
        m, c = binary_golden.meta[name], binary_golden.case(name)
        P, f, pad, s = m["P"], m["f"], m["pad"], m["stride"]
        inp = ops.pack(G(c["inp"].reshape(-1, m["cin"])), DT[bits]).view(P, m["size"], m["size"], -1)
        filt = ops.pack(G(c["filt"].reshape(-1, m["cin"])), DT[bits]).view(P, m["cout"], f, f, -1)
        filt = filt.permute(0, 2, 3, 4, 1).reshape(P, -1, m["cout"]).contiguous()    # modules/binary.py:136-137
        counts = ops.conv(inp, filt, f, f, pad, pad, s, s)
        np.testing.assert_array_equal(npy(counts), c["conv_counts"])
        act = ops.conv_act(inp, filt, G(c["thresh"]), f, f, pad, pad, s, s)
        np.testing.assert_array_equal(npy(act), c["act"])
        # the materialised-columns route of the reference gives the same numbers
        cols = ops.batch_im2col(inp, f, f, pad, pad, s, s)
        np.testing.assert_array_equal(npy(cols), B.batch_im2col(npy(inp), f, f, pad, pad, s, s))
        np.testing.assert_array_equal(npy(ops.bmm(cols, filt)).reshape(npy(counts).shape), c["conv_counts"])
        mp = ops.max_pool2d(inp, 2, 2, 0, 0, 2, 2)
        want = B.pack(c["maxpool"].reshape(-1, m["cin"]), bits).reshape(npy(mp).shape)
        np.testing.assert_array_equal(npy(mp), want)
        mp2 = ops.max_pool2d(inp, 2, 2, 1, 1, 1, 1)
        np.testing.assert_array_equal(npy(mp2), B.max_pool2d(npy(inp), 2, 2, 1, 1, 1, 1))


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("P,M,K,N", [(3, 70, 5, 9), (2, 64, 8, 64), (5, 33, 3, 1), (4, 100, 16, 1), (1, 1, 1, 1),
                                      (6, 257, 2, 1), (2, 130, 17, 70)])
def test_bmm_and_act(ops, bits, P, M, K, N):
    rng = np.random.default_rng(P * 100 + M + K + N)
    info = np.iinfo(np.int64 if bits == 64 else np.int32)
    A = rng.integers(info.min, info.max, (P, M, K), dtype=info.dtype, endpoint=True)
    Bm = rng.integers(info.min, info.max, (P, K, N), dtype=info.dtype, endpoint=True)
    want = B.bmm(A, Bm)
    got = ops.bmm(G(A), G(Bm))
    np.testing.assert_array_equal(npy(got), want)
    thresh = rng.integers(0, 2 * K * bits, (P, N)).astype(np.int32)
    np.testing.assert_array_equal(npy(ops.bmm_act(G(A), G(Bm), G(thresh))), B.bmm_act(A, Bm, thresh))


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("n,rows,cols", [(9, 6, 100), (4, 3, 64), (2, 5, 257), (3, 2, 1024)])
def test_sample_bits_injected_uniforms(ops, bits, n, rows, cols):
    rng = np.random.default_rng(n + rows + cols)
    p = rng.random((rows, cols)).astype(np.float16)
    u = rng.random((n, rows, cols)).astype(np.float32)
    u[0, 0, 0] = float(p[0, 0])            # equality is "not greater"
    got = ops.sample_bits(G(p), n, DT[bits], 0, uniforms=G(u))
    np.testing.assert_array_equal(npy(got), B.sample_bits(p, u, bits))


def test_sample_bits_philox(ops):
    p = torch.rand(64, 1000).half().to(DEV)
    a = ops.sample_bits(p, 128, torch.int64, 42)
    b = ops.sample_bits(p, 128, torch.int64, 42)
    c = ops.sample_bits(p, 128, torch.int64, 43)
    assert torch.equal(a, b) and not torch.equal(a, c)
    bits = ops.unpack(a.view(-1, a.shape[-1])).view(128, 64, -1)
    assert not bits[:, :, 1000:].any()                         # padding columns stay zero
    freq = bits[:, :, :1000].float().mean(dim=0)
    assert (freq - p.float()).abs().mean().item() < 0.05       # Bernoulli(p): sd <= .5/sqrt(128) = .044
    assert abs((freq - p.float()).mean().item()) < 0.005       # and unbiased
    assert not torch.equal(a[0], a[1])


def test_sample_bits_philox_statistics(ops):
    """Per-column frequencies over 16384 members match thresholds that need the low planes
    (p = k / 65536), the ends are exact, and neighbouring columns are uncorrelated."""
    n = 16384
    pv = torch.tensor([0.0, 1.0, 0.5, 0.25, 2.0 ** -9, 0.5 + 2.0 ** -9, 0.75, 2.0 ** -12,
                       1.0 - 2.0 ** -10, 0.3, 0.5, 0.5, 0.1, 0.9, 2.0 ** -8 + 2.0 ** -9, 0.6])
    p = pv.repeat(2, 4).half().to(DEV)                     # (2 rows, 64 columns)
    a = ops.sample_bits(p, n, torch.int32, 7)
    bits = ops.unpack(a.view(-1, a.shape[-1])).view(n, 2, 64).float()
    freq = bits.mean(dim=0).cpu()
    want = p.float().cpu()
    sd = (want * (1 - want) / n).sqrt()
    assert torch.all((freq - want).abs() <= 5 * sd + 1e-9), (freq - want).abs().max()
    assert torch.all(freq[want == 0] == 0) and torch.all(freq[want == 1] == 1)
    x = bits[:, 0, 10].cpu() - 0.5                          # p = .5 at columns 10 and 11
    y = bits[:, 0, 11].cpu() - 0.5
    assert abs(float((x * y).mean()) / 0.25) < 5 / n ** 0.5


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("D,rows,cols", [(64, 5, 100), (200, 3, 64), (33, 2, 700), (1, 1, 1),
                                         (203, 3, 1024), (37, 2, 3072), (70, 1, 9216), (3, 2, 2048)])
def test_weighted_sum(ops, bits, D, rows, cols):
    rng = np.random.default_rng(D + rows + cols)
    b = rng.integers(0, 2, (D, rows, cols)).astype(bool)
    packed = B.pack(b.reshape(-1, cols), bits).reshape(D, rows, -1)
    w = rng.standard_normal(D).astype(np.float16)
    got = npy(ops.weighted_sum(G(packed), G(w), cols)).astype(np.float64)
    want = B.weighted_sum(packed, w, cols).astype(np.float64)
    exact = np.einsum("d,dyz->yz", w.astype(np.float64), b.astype(np.float64))
    # fp32 accumulation in a different member order, then one fp16 rounding
    tol = 2.0 ** -10 * np.maximum(np.abs(exact), 1.0) + 1e-3
    assert np.all(np.abs(got - exact) <= tol)
    assert np.all(np.abs(got - want) <= 2 * tol)


def test_binarized_linear_layer(ops):
    from nesgpu_b200 import binary
    D, out_f, in_f = 16, 24, 200
    layer = binary.BinarizedLinear(in_f, out_f, D, threshold=True, device=DEV)
    with torch.no_grad():
        layer.weight.copy_(torch.randn(out_f, in_f).half())
    g = torch.Generator().manual_seed(4)
    u = torch.rand(D, out_f, in_f, generator=g)
    layer.uniforms = u.to(DEV)
    layer.set_seed(9)
    layer.set_noise()
    P = npy(layer.bernoulli_probabilities())
    # fp16 mean / division may round differently on the two devices: one fp16 step of slack
    np.testing.assert_allclose(P.astype(np.float32), B.bernoulli_probabilities(npy(layer.weight)).astype(np.float32),
                               atol=2e-3)
    wbits = B.sample_bits(P, u.numpy(), 64)
    np.testing.assert_array_equal(npy(layer.weight_noise), wbits)
    x = torch.randint(2, (D, in_f), generator=g).bool()
    layer.perturbed_flag = True
    layer.threshold = False
    act = layer.forward(x.to(DEV))
    np.testing.assert_array_equal(npy(act), B.binarized_linear_forward(wbits, x.numpy(), in_f))
    layer.threshold = True
    got = layer.forward(x.to(DEV))
    thresh = (layer.bias + layer.bias_noise).detach().float().cpu().numpy()
    np.testing.assert_array_equal(npy(got), B.binarized_linear_forward(wbits, x.numpy(), in_f) > thresh)
    layer.update(torch.randn(D, device=DEV))
    assert layer.weight.grad.shape == (out_f, in_f) and layer.weight.grad.dtype == torch.float16
    assert layer.bias.grad.shape == (out_f,)


def test_binarized_conv_and_pool_layers(ops):
    from nesgpu_b200 import binary
    D, cin, cout, size = 6, 70, 5, 9
    conv = binary.BinarizedConv2d(cin, cout, D, 3, padding=1, threshold=False, device=DEV)
    with torch.no_grad():
        conv.weight.copy_(torch.randn_like(conv.weight))
    conv.set_seed(1)
    conv.set_noise()
    x = torch.randint(2, (D, size, size, cin)).bool()
    conv.perturbed_flag = True
    got = conv.forward(x.to(DEV))
    wb = npy(conv.weight_noise).reshape(D, cout, 3, 3, -1).transpose(0, 2, 3, 4, 1).reshape(D, -1, cout)
    xin = B.pack(x.numpy().reshape(-1, cin), 64).reshape(D, size, size, -1)
    want = 2 * B.conv(xin, wb, 3, 3, 1, 1, 1, 1) - cin * 9
    np.testing.assert_array_equal(npy(got), want)
    pool = binary.BinarizedMaxPool2d()
    np.testing.assert_array_equal(npy(pool(x.to(DEV))), B.max_pool2d(xin, 2, 2, 0, 0, 2, 2))


def test_config4_binary_layer_full_size(ops):
    """population 1024, 1024x1024 weights, one 1024-bit input vector per member."""
    D = n = 1024
    g = torch.Generator().manual_seed(1004)
    p = torch.rand(n, n, generator=g).half()
    # weight bits for a slice of members with injected uniforms (bit-exact) ...
    u = torch.rand(16, n, n, generator=g)
    u = u.clamp_min(2.0 ** -24)
    got = ops.sample_bits(p.to(DEV), 16, torch.int64, 0, uniforms=u.to(DEV))
    np.testing.assert_array_equal(npy(got), B.sample_bits(p.numpy(), u.numpy(), 64))
    # ... and the full population from the device generator
    wbits = ops.sample_bits(p.to(DEV), D, torch.int64, 77)
    assert wbits.shape == (D, n, 16)
    x = torch.randint(2, (D, n), generator=g).bool()
    xb = ops.pack(x.to(DEV), torch.int64)
    np.testing.assert_array_equal(npy(xb), B.pack(x.numpy(), 64))
    counts = ops.bmm(wbits, xb.view(D, -1, 1))
    np.testing.assert_array_equal(npy(counts), B.bmm(npy(wbits), npy(xb).reshape(D, -1, 1)))
    # general-N path on the same data agrees with the N = 1 fast path
    xb4 = xb.view(D, -1, 1).repeat(1, 1, 4).contiguous()
    assert torch.equal(ops.bmm(wbits, xb4)[:, :, 2], counts[:, :, 0])
    # weighted sum at full size: compare 8 output rows against the oracle
    w = torch.randn(D, generator=g).half()
    ws = ops.weighted_sum(wbits, w.to(DEV), n)
    sub = npy(wbits)[:, 100:108, :]
    want = B.weighted_sum(sub, w.numpy(), n).astype(np.float64)
    assert np.all(np.abs(npy(ws)[100:108].astype(np.float64) - want) <= 2.0 ** -9 * np.maximum(np.abs(want), 1.0) + 2e-3)
    mp_in = torch.randint(-2 ** 62, 2 ** 62, (D, 32, 32, 1), generator=g)
    np.testing.assert_array_equal(npy(ops.max_pool2d(mp_in.to(DEV), 2, 2, 0, 0, 2, 2)),
                                  B.max_pool2d(mp_in.numpy(), 2, 2, 0, 0, 2, 2))


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("n,rows,cols", [(40, 33, 1024), (5, 7, 100), (17, 3, 2048), (1, 1, 1)])
def test_seeded_bmv_equals_sample_then_bmm(ops, bits, n, rows, cols):
    g = torch.Generator().manual_seed(n + rows + cols)
    p = torch.rand(rows, cols, generator=g).half().to(DEV)
    x = torch.randint(2, (n, cols), generator=g).bool().to(DEV)
    xb = ops.pack(x, DT[bits])
    fused = ops.binary_seeded_bmv(p, xb, 1234)
    stored = ops.bmm(ops.sample_bits(p, n, DT[bits], 1234), xb.view(n, -1, 1)).squeeze(2)
    assert torch.equal(fused, stored)
    assert not torch.equal(fused, ops.binary_seeded_bmv(p, xb, 1235)) or n * rows * cols < 64


# ------------------------------------------------------------------ layer arithmetic behind the C ABI

def _linear_layer(binary, D, out_f, in_f, batch_norm, seed, dtype=torch.int64):
    layer = binary.BinarizedLinear(in_f, out_f, D, threshold=True, batch_norm=batch_norm, dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        layer.weight.copy_(torch.randn(out_f, in_f, generator=g).half())
        layer.bias.copy_((4 * torch.randn(out_f, generator=g)).half())
    layer.set_seed(seed)
    layer.set_noise()
    layer.perturbed_flag = True
    return layer, g


@pytest.mark.parametrize("D,out_f,in_f,bits", [(16, 24, 256, 64), (40, 100, 1024, 64), (9, 33, 128, 32), (5, 70, 4096, 64)])
@pytest.mark.parametrize("batch_norm", [False, True])
def test_binarized_linear_thresholds_and_packed_output(ops, D, out_f, in_f, bits, batch_norm):
    """One streaming kernel (two more launches with the batch mean): bit-exact against the restated layer, as bools
    and as packed words; the fp16 steps are the reference's (int32 activation compared in fp16)."""
    from nesgpu_b200 import binary
    layer, g = _linear_layer(binary, D, out_f, in_f, batch_norm, seed=D + out_f, dtype=DT[bits])
    x = torch.randint(2, (D, in_f), generator=g).bool()
    wbits, beta, bias = npy(layer.weight_noise), npy(layer.bias_noise), npy(layer.bias)
    want = B.binarized_linear_layer(wbits, x.numpy(), in_f, bias, beta, batch_norm, bits)
    got = layer.forward(x.to(DEV))
    assert got.dtype == torch.bool
    np.testing.assert_array_equal(npy(got), want)
    layer.packed_output = True
    packed = layer.forward(ops.pack(x.to(DEV), DT[bits]))         # packed input, packed output
    np.testing.assert_array_equal(npy(packed), B.pack(want, bits))
    layer.threshold = False
    np.testing.assert_array_equal(npy(layer.forward(x.to(DEV))), B.binarized_linear_forward(wbits, x.numpy(), in_f, None, bits))


def test_binarized_linear_rows_that_are_not_whole_chunks(ops):
    """in_features = 200 with int32 words: 7 words = 28 bytes per row, the tiled product + shared epilogue path."""
    from nesgpu_b200 import binary
    layer, g = _linear_layer(binary, 6, 10, 200, False, seed=3, dtype=torch.int32)
    x = torch.randint(2, (6, 200), generator=g).bool()
    want = B.binarized_linear_layer(npy(layer.weight_noise), x.numpy(), 200, npy(layer.bias), npy(layer.bias_noise), False, 32)
    np.testing.assert_array_equal(npy(layer.forward(x.to(DEV))), want)


@pytest.mark.parametrize("batch_norm", [False, True])
def test_binarized_conv_thresholds(ops, batch_norm):
    from nesgpu_b200 import binary
    D, cin, cout, size = 5, 96, 40, 8
    conv = binary.BinarizedConv2d(cin, cout, D, 3, padding=1, threshold=True, batch_norm=batch_norm, device=DEV)
    g = torch.Generator().manual_seed(12)
    with torch.no_grad():
        conv.weight.copy_(torch.randn(conv.weight.shape, generator=g).half())
        conv.bias.copy_((6 * torch.randn(cout, generator=g)).half())
    conv.set_seed(2)
    conv.set_noise()
    conv.perturbed_flag = True
    x = torch.randint(2, (D, size, size, cin), generator=g).bool()
    wb = npy(conv.weight_noise).reshape(D, cout, 3, 3, -1).transpose(0, 2, 3, 4, 1).reshape(D, -1, cout)
    xin = B.pack(x.numpy().reshape(-1, cin), 64).reshape(D, size, size, -1)
    counts = B.conv(xin, wb, 3, 3, 1, 1, 1, 1)
    want = B.binarized_conv_layer(counts, cin * 9, npy(conv.bias), npy(conv.bias_noise), batch_norm)
    got = conv.forward(x.to(DEV))
    np.testing.assert_array_equal(npy(got), want)
    conv.packed_output = True
    packed = conv.forward(x.to(DEV))
    # packed NHWC words for the next layer
    np.testing.assert_array_equal(npy(packed), B.pack(want.reshape(-1, cout), 64).reshape(D, size, size, -1))


def test_binarized_update_matches_the_restated_layer(ops):
    from nesgpu_b200 import binary
    layer, g = _linear_layer(binary, 64, 48, 256, False, seed=8)
    fitness = torch.randn(64, generator=g)
    layer.update(fitness.to(DEV), l1=0.01, l2=0.02)
    wg, bg = B.binarized_update(npy(layer.weight_noise), fitness.numpy(), npy(layer.weight), npy(layer.bias_noise), 256,
                                l1=0.01, l2=0.02)
    got_w, got_b = npy(layer.weight.grad).astype(np.float64), npy(layer.bias.grad).astype(np.float64)
    # fp16 results of fp32 sums taken in another order: one fp16 rounding step of slack
    assert np.all(np.abs(got_w - wg.astype(np.float64)) <= 2.0 ** -9 * np.maximum(np.abs(wg.astype(np.float64)), 1.0) + 2e-3)
    assert np.all(np.abs(got_b - bg.astype(np.float64)) <= 2.0 ** -9 * np.maximum(np.abs(bg.astype(np.float64)), 1.0) + 2e-3)


def test_binarized_noise_statistics_and_probabilities(ops):
    from nesgpu_b200 import binary
    layer, _ = _linear_layer(binary, 256, 64, 512, False, seed=6)
    bn = layer.bias_noise.float()
    assert bn.min().item() >= -3.0 and bn.max().item() < 3.0
    assert abs(bn.mean().item()) < 0.05 and abs(bn.std().item() - 3 ** .5) < 0.05      # uniform on [-3, 3)
    P = npy(layer.bernoulli_probabilities()).astype(np.float32)
    np.testing.assert_allclose(P, B.bernoulli_probabilities(npy(layer.weight)).astype(np.float32), atol=2e-3)
    other = binary.BinarizedLinear(512, 64, 256, device=DEV)
    other.set_seed(6)
    other.set_member_offset(256)
    other.set_noise()
    assert not torch.equal(other.bias_noise, layer.bias_noise)
