"""The CPU oracle against the golden vectors produced by the reference itself
(tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import binary_ref as B
from oracle import perturbed_ref as O

TOL = dict(rtol=1e-5, atol=1e-5)


def T(a):
    return None if a is None else torch.from_numpy(np.asarray(a))


def test_perturbed_linear(perturbed_golden):
    for name in perturbed_golden.names("PerturbedLinear"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        y = O.perturbed_linear_forward(T(c["x"]), T(c["weight"]), T(c.get("bias")), T(c["weight_noise"]),
                                       T(c.get("bias_noise")), m["D"], m["antithetic"], m["direct"])
        np.testing.assert_allclose(y.numpy(), c["y"], **TOL)
        noise = T(c["weight_noise"])
        bnoise = T(c.get("bias_noise"))
        if m["direct"]:
            noise = noise - T(c["weight"])
            bnoise = bnoise - T(c["bias"])
        g, bg = O.perturbed_update(T(c["weight"]), noise, bnoise, T(c["w"]), m["l1"], m["l2"])
        np.testing.assert_allclose(g.numpy(), c["grad"], **TOL)
        if m["bias"]:
            np.testing.assert_allclose(bg.numpy(), c["bias_grad"], **TOL)


def test_perturbed_conv(perturbed_golden):
    for name in perturbed_golden.names("PerturbedConv2d"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        y = O.perturbed_conv2d_forward(T(c["x"]), T(c["weight"]), T(c["bias"]), T(c["weight_noise"]),
                                       T(c["bias_noise"]), m["D"], m["stride"], m["padding"], 1,
                                       m["antithetic"])
        np.testing.assert_allclose(y.numpy(), c["y"], **TOL)
        g, bg = O.perturbed_update(T(c["weight"]), T(c["weight_noise"]), T(c["bias_noise"]), T(c["w"]))
        np.testing.assert_allclose(g.numpy(), c["grad"], **TOL)
        np.testing.assert_allclose(bg.numpy(), c["bias_grad"], **TOL)


def test_permuted_linear(perturbed_golden):
    for name in perturbed_golden.names("PermutedLinear"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        y = O.permuted_linear_forward(T(c["x"]), T(c["weight"]), T(c["bias"]), T(c["weight_noise"]),
                                      T(c["bias_noise"]), T(c.get("pin")), T(c.get("pout")), m["D"],
                                      m["antithetic"])
        np.testing.assert_allclose(y.numpy(), c["y"], **TOL)
        # the dense-equivalent form gives the same forward through the IID layer
        E = O.dense_member_noise(T(c["weight_noise"]), T(c.get("pin")), T(c.get("pout")), m["in_f"], m["out_f"])
        y2 = O.perturbed_linear_forward(T(c["x"]), T(c["weight"]), T(c["bias"]), E, T(c["bias_noise"]),
                                        m["D"], m["antithetic"])
        np.testing.assert_allclose(y2.numpy(), c["y"], **TOL)
        if "perm_weights" in c:
            pw = O.permutation_weights(T(c["w"]), T(c.get("pin")), T(c.get("pout")), m["in_f"], m["out_f"],
                                       m["in_sp"], m["out_sp"])
            np.testing.assert_allclose(pw.numpy(), c["perm_weights"], **TOL)
        if "grad" in c:
            g = O.permuted_linear_weight_grad(T(c["weight_noise"]), T(c["w"]), T(c.get("pin")),
                                              T(c.get("pout")), m["in_f"], m["out_f"])
            np.testing.assert_allclose(g.numpy(), c["grad"], **TOL)


def test_permuted_conv(perturbed_golden):
    for name in perturbed_golden.names("PermutedConv2d"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        y = O.permuted_conv2d_forward(T(c["x"]), T(c["weight"]), T(c["bias"]), T(c["weight_noise"]),
                                      T(c["bias_noise"]), T(c.get("pin")), T(c.get("pout")), m["D"],
                                      m["stride"], m["padding"], 1, m["antithetic"])
        np.testing.assert_allclose(y.numpy(), c["y"], **TOL)
        g = O.permuted_conv2d_weight_grad(T(c["weight_noise"]), T(c["w"]), T(c.get("pin")), T(c.get("pout")),
                                          m["cin"], m["cout"])
        np.testing.assert_allclose(g.numpy(), c["grad"], **TOL)
        # dense-equivalent noise through the IID conv gives the same forward
        E = O.dense_member_noise(T(c["weight_noise"]), T(c.get("pin")), T(c.get("pout")), m["cin"], m["cout"])
        y2 = O.perturbed_conv2d_forward(T(c["x"]), T(c["weight"]), T(c["bias"]), E, T(c["bias_noise"]),
                                        m["D"], m["stride"], m["padding"], 1, m["antithetic"])
        np.testing.assert_allclose(y2.numpy(), c["y"], **TOL)


def test_constructor_rule(perturbed_golden):
    for rule in perturbed_golden.meta["__constructor_rules__"]:
        assert list(O.resolve_permutation(*rule["args"])) == rule["result"], rule


def test_sparse_is_dense_equivalent():
    g = torch.Generator().manual_seed(3)
    D, out_f, in_f, k = 4, 6, 9, 2
    idx = torch.randint(in_f, (D, out_f, k), generator=g)
    val = torch.randn(D, out_f, k, generator=g)
    x = torch.randn(2 * D, in_f, generator=g)
    W = torch.randn(out_f, in_f, generator=g)
    y = O.sparse_perturbed_linear_forward(x, W, None, idx, val, None, D, True)
    for b in range(2 * D):
        d, r = b % D, b // D
        s = -1.0 if r >= 1 else 1.0
        for o in range(out_f):
            ref = x[b] @ W[o] + s * sum(x[b, idx[d, o, t]] * val[d, o, t] for t in range(k))
            assert abs(float(ref) - float(y[b, o])) < 1e-5


@pytest.mark.parametrize("bits", [32, 64])
def test_binary_conv_pool(binary_golden, bits):
    for name in binary_golden.names():
        m, c = binary_golden.meta[name], binary_golden.case(name)
        P, f, pad, s = m["P"], m["f"], m["pad"], m["stride"]
        inp = B.pack(c["inp"].reshape(-1, m["cin"]), bits).reshape(P, m["size"], m["size"], -1)
        filt = B.pack(c["filt"].reshape(-1, m["cin"]), bits).reshape(P, m["cout"], f, f, -1)
        filt = filt.transpose(0, 2, 3, 4, 1).reshape(P, -1, m["cout"])   # modules/binary.py:136-137
        counts = B.conv(inp, filt, f, f, pad, pad, s, s)
        np.testing.assert_array_equal(counts, c["conv_counts"])
        act = B.conv_act(inp, filt, c["thresh"], f, f, pad, pad, s, s)
        np.testing.assert_array_equal(act, c["act"])
        mp = B.max_pool2d(inp, 2, 2, 0, 0, 2, 2)
        want = B.pack(c["maxpool"].reshape(-1, m["cin"]), bits).reshape(mp.shape)
        np.testing.assert_array_equal(mp, want)


def test_binary_pack_roundtrip_and_layouts():
    rng = np.random.default_rng(5)
    b = rng.integers(0, 2, (7, 150)).astype(bool)
    for bits in (32, 64):
        w = B.pack(b, bits)
        assert w.shape == (7, (150 + bits - 1) // bits)
        np.testing.assert_array_equal(B.unpack(w, bits)[:, :150], b)
        assert not B.unpack(w, bits)[:, 150:].any()
    # LSB-first (pack.cu:25-27)
    one = np.zeros((1, 64), bool)
    one[0, 3] = True
    assert B.pack(one, 64)[0, 0] == 8
    top = np.zeros((1, 64), bool)
    top[0, 63] = True
    assert B.pack(top, 64)[0, 0] == np.iinfo(np.int64).min
    # int8pack == pack of the unpacked bytes (booloptests.py:142-144, commented check)
    by = rng.integers(0, 256, (5, 19)).astype(np.uint8)
    bits_of = ((by[..., None] >> np.arange(8)) & 1).astype(bool).reshape(5, -1)
    np.testing.assert_array_equal(B.int8pack(by, 64), B.pack(bits_of, 64))
    np.testing.assert_array_equal(B.pack8(b).view(np.uint8),
                                  np.packbits(np.pad(b, ((0, 0), (0, 2))), axis=1, bitorder="little"))


def test_binary_linear_is_negated_dot():
    rng = np.random.default_rng(9)
    D, out_f, in_f = 3, 5, 130
    wb = rng.integers(0, 2, (D, out_f, in_f)).astype(bool)
    xb = rng.integers(0, 2, (D, in_f)).astype(bool)
    wbits = B.pack(wb.reshape(-1, in_f), 64).reshape(D, out_f, -1)
    act = B.binarized_linear_forward(wbits, xb, in_f)
    pm = lambda a: 2 * a.astype(np.int32) - 1
    want = -np.einsum("doi,di->do", pm(wb), pm(xb))
    np.testing.assert_array_equal(act, want)


def test_binary_sample_and_weighted_sum():
    rng = np.random.default_rng(11)
    p = rng.random((6, 100)).astype(np.float16)
    u = rng.random((9, 6, 100)).astype(np.float32)
    bits = B.sample_bits(p, u, 64)
    assert bits.shape == (9, 6, 2)
    np.testing.assert_array_equal(B.unpack(bits.reshape(-1, 2), 64).reshape(9, 6, 128)[:, :, :100],
                                  p.astype(np.float32) > u)
    w = rng.standard_normal(9).astype(np.float16)
    ws = B.weighted_sum(bits, w, 100)
    want = np.einsum("d,dyz->yz", w.astype(np.float64), (p.astype(np.float32) > u).astype(np.float64))
    np.testing.assert_allclose(ws.astype(np.float64), want, atol=2e-2)


def test_synthetic_layers(perturbed_golden):
    for name in perturbed_golden.names("SyntheticLinear"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        fin, fout = T(c.get("fin")), T(c.get("fout"))
        y = O.synthetic_linear_forward(T(c["x"]), T(c["weight"]), T(c["bias"]), T(c["weight_noise"]), T(c["bias_noise"]),
                                       fin, fout, m["D"], m["antithetic"])
        np.testing.assert_allclose(y.numpy(), c["y"], **TOL)
        if "grad" in c:
            g = O.synthetic_weight_grad(T(c["weight_noise"]), T(c["w"]), fin, fout)
            np.testing.assert_allclose(g.numpy(), c["grad"], **TOL)
    for name in perturbed_golden.names("SyntheticConv2d"):
        m, c = perturbed_golden.meta[name], perturbed_golden.case(name)
        fin, fout = T(c.get("fin")), T(c.get("fout"))
        y = O.synthetic_conv2d_forward(T(c["x"]), T(c["weight"]), T(c["bias"]), T(c["weight_noise"]), T(c["bias_noise"]),
                                       fin, fout, m["D"], m["stride"], m["padding"], 1, m["antithetic"])
        np.testing.assert_allclose(y.numpy(), c["y"], **TOL)
        if "grad" in c:
            g = O.synthetic_weight_grad(T(c["weight_noise"]), T(c["w"]), fin, fout)
            np.testing.assert_allclose(g.numpy(), c["grad"], **TOL)
    # two-sided gradient equals sum_d w_d E_d with E_d = f_out f_in^T * eps
    g = torch.Generator().manual_seed(2)
    D, out_f, in_f = 5, 4, 6
    eps = torch.randn(out_f, in_f, generator=g)
    fo = (2 * torch.randint(2, (D, out_f), generator=g) - 1).to(torch.int8)
    fi = (2 * torch.randint(2, (D, in_f), generator=g) - 1).to(torch.int8)
    w = torch.randn(D, generator=g)
    E = fo.float().unsqueeze(2) * fi.float().unsqueeze(1) * eps
    np.testing.assert_allclose(O.synthetic_weight_grad(eps, w, fi, fo).numpy(), torch.einsum("d,dkm->km", w, E).numpy(), **TOL)
