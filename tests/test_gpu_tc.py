"""Tensor-core (tcgen05 / TMA) GEMM against a float64 CPU product.

Tolerances: mode 3 (3xTF32, error-compensated) must hold the fp32 bar (rel err <= 1e-4; it measures
~1e-6); mode 1 (plain TF32) is the stated reduced-precision mode with the 2e-2 bar (it measures ~5e-4)."""
import pytest
import torch

from gpu_util import DEV, G, assert_close, rel_err

pytestmark = pytest.mark.gpu


def _run(C, x, w, b, mode):
    M, K = x.shape
    N = w.shape[0]
    y = torch.full((M, N), float("nan"), device=DEV)
    nbytes = C.call("nes_linear_fwd_tc_scratch_bytes", M, N, K, mode)
    buf = torch.empty(nbytes + 256, dtype=torch.uint8, device=DEV)
    off = (-buf.data_ptr()) % 256
    C.call("nes_linear_fwd_tc", C.ptr(x), C.ptr(w), C.ptr(b), C.ptr(y), M, N, K, mode,
           buf.data_ptr() + off, nbytes, C.stream())
    torch.cuda.synchronize()
    return y


def _flag(C):
    import ctypes
    v = ctypes.c_int(-1)
    C.call("nes_tc_error_flag", ctypes.byref(v))
    return v.value


@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (128, 128, 256), (256, 384, 64), (200, 136, 100),
                                   (1, 1, 4), (130, 257, 36), (2048, 1024, 1024)])
def test_linear_tc_modes(M, N, K):
    from nesgpu_b200 import _cabi as C
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) / K ** .5
    b = torch.randn(N, generator=g)
    want = (x.double() @ w.double().t() + b.double()).float()
    y3 = _run(C, x.to(DEV), w.to(DEV), b.to(DEV), 3)
    assert _flag(C) == 0
    e3 = rel_err(y3, want)
    assert e3 <= 1e-5, "3xTF32 rel err %g" % e3
    y1 = _run(C, x.to(DEV), w.to(DEV), None, 1)
    assert _flag(C) == 0
    e1 = rel_err(y1, (x.double() @ w.double().t()).float())
    assert e1 <= 5e-3, "TF32 rel err %g" % e1


def test_linear_tc_rejects_unaligned_k():
    from nesgpu_b200 import _cabi as C
    x = torch.zeros(4, 6, device=DEV)
    w = torch.zeros(4, 6, device=DEV)
    y = torch.zeros(4, 4, device=DEV)
    buf = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    with pytest.raises(NotImplementedError):
        C.call("nes_linear_fwd_tc", C.ptr(x), C.ptr(w), None, C.ptr(y), 4, 4, 6, 3, C.ptr(buf), 4096, C.stream())


# ------------------------------------------------------------------ tensor-core convolutions (TF32 mode)
# Stated reduced-precision mode: operands rounded to TF32.  Bar 2e-2; measured ~5e-4.
TC_CONV_TOL = 5e-3


def _perms(g, D, n, keep=None):
    p = torch.stack([torch.randperm(n, generator=g) for _ in range(D)]).short()
    return p[:, :keep].contiguous() if keep else p


@pytest.mark.parametrize("mode,in_sp,out_sp,R,anti,hw,k,pad,cin", [
    ("out", 0, 0.5, 1, False, 13, 3, 1, 64), ("in", 0, 0, 2, True, 9, 3, 1, 64), ("both", 0, 0, 3, True, 8, 3, 0, 64),
    ("out", 0, 0, 2, True, 33, 1, 0, 64), ("auto", 0.5, 0, 1, False, 20, 5, 2, 32),
])
def test_permuted_conv_tf32(mode, in_sp, out_sp, R, anti, hw, k, pad, cin):
    from nesgpu_b200 import base, _cabi as C
    from oracle import perturbed_ref as O
    from gpu_util import G, set_params
    D, cout = 5, 32
    g = torch.Generator().manual_seed(hw + k)
    layer = base.PermutedConv2d(cin, cout, k, D, padding=pad, antithetic=anti, permutation=mode, in_sparsity=in_sp,
                                out_sparsity=out_sp, options={"tc": "tf32"}).to(DEV)
    isp, osp = layer.in_sparsity, layer.out_sparsity
    x = torch.randn(R * D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g)
    eps = 0.05 * torch.randn(osp, isp, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g)
    pin = _perms(g, D, cin, isp) if layer.permute_inputs else None
    pout = _perms(g, D, cout) if layer.permute_outputs else None
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(eps), G(beta)
    layer.input_permutations, layer.output_permutations = G(pin), G(pout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    torch.cuda.synchronize()
    assert _flag(C) == 0
    want = O.permuted_conv2d_forward(x, W, b, eps, beta, pin, pout, D, 1, pad, 1, anti)
    e = rel_err(y, want)
    assert e <= TC_CONV_TOL, "TF32 conv rel err %g" % e


def test_perturbed_conv_tf32():
    from nesgpu_b200 import base, _cabi as C
    from oracle import perturbed_ref as O
    from gpu_util import G, set_params
    D, R, cin, cout, hw, k = 4, 2, 32, 64, 12, 3
    g = torch.Generator().manual_seed(23)
    x = torch.randn(R * D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g)
    E = 0.05 * torch.randn(D, cout, cin, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g)
    layer = base.PerturbedConv2d(cin, cout, k, D, padding=1, antithetic=True, options={"tc": "tf32"}).to(DEV)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(E), G(beta)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    torch.cuda.synchronize()
    assert _flag(C) == 0
    e = rel_err(y, O.perturbed_conv2d_forward(x, W, b, E, beta, D, 1, 1, 1, True))
    assert e <= TC_CONV_TOL, "TF32 conv rel err %g" % e


def test_config3_permuted_conv_tf32_full_size():
    from nesgpu_b200 import base, _cabi as C
    from oracle import perturbed_ref as O
    from gpu_util import G, set_params
    D, c, hw = 1024, 64, 32
    g = torch.Generator().manual_seed(1003)
    layer = base.PermutedConv2d(c, c, 3, D, padding=1, out_sparsity=.5, options={"tc": "tf32"}).to(DEV)
    x = torch.randn(D, c, hw, hw, generator=g)
    W = torch.randn(c, c, 3, 3, generator=g) * (2 / 576) ** .5
    b = torch.zeros(c)
    eps = 0.02 * 2 ** .5 * torch.randn(32, c, 3, 3, generator=g)
    beta = 0.02 * torch.randn(D, c, generator=g)
    pout = _perms(g, D, c)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.output_permutations = G(eps), G(beta), G(pout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    torch.cuda.synchronize()
    assert _flag(C) == 0
    want = O.permuted_conv2d_forward(x, W, b, eps, beta, None, pout, D, 1, 1, 1, False)
    e = rel_err(y, want)
    assert e <= TC_CONV_TOL, "TF32 conv rel err %g" % e
    # the member-to-member signal survives the rounding: compare the perturbation term on its own scale
    basey = torch.nn.functional.conv2d(x[:16], W, b, 1, 1)
    e2 = rel_err(y[:16].cpu() - basey, want[:16] - basey)
    assert e2 <= 2e-2, "TF32 perturbation-term rel err %g" % e2


def test_conv_tc_rejects_unsupported_shapes():
    from nesgpu_b200 import base
    layer = base.PermutedConv2d(3, 32, 3, 4, options={"tc": "tf32"}).to(DEV)
    layer.set_noise(0.02)
    layer.perturbed_flag = True
    with pytest.raises(NotImplementedError):
        layer.forward(torch.zeros(4, 3, 8, 8, device=DEV))


# ------------------------------------------------------------------ bf16 tensor-core convolutions
# Stated reduced-precision mode: operands rounded to bf16 (8 mantissa bits), fp32 accumulation.  Bar 2e-2.
BF16_CONV_TOL = 1e-2


@pytest.mark.parametrize("mode,in_sp,out_sp,R,anti,hw,k,pad,cout", [
    ("out", 0, 0.5, 1, False, 13, 3, 1, 64), ("in", 0, 0, 2, True, 9, 3, 1, 32), ("both", 0, 0, 3, True, 8, 3, 0, 64),
    ("out", 0, 0, 2, True, 33, 1, 0, 128), ("auto", 0.5, 0, 1, False, 20, 3, 2, 24),
])
def test_permuted_conv_bf16(mode, in_sp, out_sp, R, anti, hw, k, pad, cout):
    from nesgpu_b200 import base, _cabi as C
    from oracle import perturbed_ref as O
    from gpu_util import G, set_params
    D, cin = 5, 64
    g = torch.Generator().manual_seed(hw + k)
    layer = base.PermutedConv2d(cin, cout, k, D, padding=pad, antithetic=anti, permutation=mode, in_sparsity=in_sp,
                                out_sparsity=out_sp, options={"tc": "bf16"}).to(DEV)
    isp, osp = layer.in_sparsity, layer.out_sparsity
    x = torch.randn(R * D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g)
    eps = 0.05 * torch.randn(osp, isp, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g)
    pin = _perms(g, D, cin, isp) if layer.permute_inputs else None
    pout = _perms(g, D, cout) if layer.permute_outputs else None
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(eps), G(beta)
    layer.input_permutations, layer.output_permutations = G(pin), G(pout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    torch.cuda.synchronize()
    assert _flag(C) == 0
    e = rel_err(y, O.permuted_conv2d_forward(x, W, b, eps, beta, pin, pout, D, 1, pad, 1, anti))
    assert e <= BF16_CONV_TOL, "bf16 conv rel err %g" % e


def test_perturbed_conv_bf16():
    from nesgpu_b200 import base, _cabi as C
    from oracle import perturbed_ref as O
    from gpu_util import G, set_params
    D, R, cin, cout, hw, k = 4, 2, 64, 64, 12, 3
    g = torch.Generator().manual_seed(29)
    x = torch.randn(R * D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g)
    E = 0.05 * torch.randn(D, cout, cin, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g)
    layer = base.PerturbedConv2d(cin, cout, k, D, padding=1, antithetic=True, options={"tc": "bf16"}).to(DEV)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(E), G(beta)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    torch.cuda.synchronize()
    assert _flag(C) == 0
    e = rel_err(y, O.perturbed_conv2d_forward(x, W, b, E, beta, D, 1, 1, 1, True))
    assert e <= BF16_CONV_TOL, "bf16 conv rel err %g" % e


def test_config3_permuted_conv_bf16_full_size():
    from nesgpu_b200 import base, _cabi as C
    from oracle import perturbed_ref as O
    from gpu_util import G, set_params
    D, c, hw = 1024, 64, 32
    g = torch.Generator().manual_seed(1003)
    layer = base.PermutedConv2d(c, c, 3, D, padding=1, out_sparsity=.5, options={"tc": "bf16"}).to(DEV)
    x = torch.randn(D, c, hw, hw, generator=g)
    W = torch.randn(c, c, 3, 3, generator=g) * (2 / 576) ** .5
    b = torch.zeros(c)
    eps = 0.02 * 2 ** .5 * torch.randn(32, c, 3, 3, generator=g)
    beta = 0.02 * torch.randn(D, c, generator=g)
    pout = _perms(g, D, c)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.output_permutations = G(eps), G(beta), G(pout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    torch.cuda.synchronize()
    assert _flag(C) == 0
    want = O.permuted_conv2d_forward(x, W, b, eps, beta, None, pout, D, 1, 1, 1, False)
    e = rel_err(y, want)
    assert e <= BF16_CONV_TOL, "bf16 conv rel err %g" % e


# ---- PermutedLinear as one tensor-core product ----------------------------------------------------

@pytest.mark.parametrize("tc,tol", [("bf16x3", 1e-4), ("3xtf32", 1e-4), ("tf32", 2e-2), ("bf16", 2e-2)])
@pytest.mark.parametrize("mode,in_sp,out_sp,R,anti,in_f,out_f,bias", [
    ("in", 0, 0, 2, True, 200, 136, True), ("in", 0.1, 0, 3, True, 203, 70, True),
    ("in", 0, 0, 1, False, 64, 10, False), ("in", 0.5, 0, 4, True, 1600, 128, True),
])
def test_permuted_linear_single_product(tc, tol, mode, in_sp, out_sp, R, anti, in_f, out_f, bias):
    """options["tc"] forces the one-product form; split-bf16 and 3xTF32 hold the fp32 bar, TF32 and bf16 are the stated 2e-2 modes."""
    from nesgpu_b200 import base
    from oracle import perturbed_ref as O
    from gpu_util import G, set_params
    D = 48
    g = torch.Generator().manual_seed(in_f + out_f + R)
    layer = base.PermutedLinear(in_f, out_f, D, bias=bias, antithetic=anti, permutation=mode, in_sparsity=in_sp,
                                out_sparsity=out_sp, options={"tc": tc}).to(DEV)
    isp, osp = layer.in_sparsity, layer.out_sparsity
    assert layer.permute_inputs and not layer.permute_outputs
    x = torch.randn(R * D, in_f, generator=g)
    W = torch.randn(out_f, in_f, generator=g) / in_f ** .5
    b = torch.randn(out_f, generator=g) if bias else None
    eps = 0.05 * torch.randn(osp, isp, generator=g)
    beta = 0.02 * torch.randn(D, out_f, generator=g) if bias else None
    pin = torch.stack([torch.randperm(in_f, generator=g)[:isp] for _ in range(D)]).short()
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(eps), (G(beta) if bias else None)
    layer.input_permutations = G(pin)
    before = C_launches()
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    assert C_launches() - before == 3                       # operand pre-pass, filter pre-pass, tile kernel
    want = O.permuted_linear_forward(x, W, b if bias else torch.zeros(out_f), eps,
                                     beta if bias else torch.zeros(D, out_f), pin, None, D, anti)
    assert rel_err(y, want) <= tol
    assert _flag(_C()) == 0


def test_permuted_linear_auto_takes_single_product_for_large_batches():
    from nesgpu_b200 import base
    from oracle import perturbed_ref as O
    from gpu_util import G, set_params
    D, R, in_f, out_f = 512, 16, 96, 128
    g = torch.Generator().manual_seed(3)
    layer = base.PermutedLinear(in_f, out_f, D, antithetic=True, permutation="in").to(DEV)
    x = torch.randn(R * D, in_f, generator=g)
    W = torch.randn(out_f, in_f, generator=g) / in_f ** .5
    b = torch.randn(out_f, generator=g)
    eps = 0.05 * torch.randn(out_f, in_f, generator=g)
    beta = 0.02 * torch.randn(D, out_f, generator=g)
    pin = torch.stack([torch.randperm(in_f, generator=g) for _ in range(D)]).short()
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.input_permutations = G(eps), G(beta), G(pin)
    assert layer._single_product_mode(R * D, None) == 4 and layer._single_product_mode(64, None) == 0
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    assert rel_err(y, O.permuted_linear_forward(x, W, b, eps, beta, pin, None, D, True)) <= 1e-4


def _C():
    from nesgpu_b200 import _cabi
    return _cabi


def C_launches():
    return _C().call("nes_launch_count")


# ---- out-permuted conv + ReLU + MaxPool2d(2) in one tensor-core kernel ------------------------------

@pytest.mark.parametrize("cout,out_sp,hw,k,R,anti,bias,D", [
    (64, 0, 13, 3, 2, False, True, 5),        # second layer of the small CNN
    (64, 0.5, 13, 3, 4, True, True, 3),       # half of the channels carry noise, antithetic halves
    (40, 0, 12, 3, 1, False, False, 7),       # fewer channels, even output, no bias
    (64, 0, 10, 2, 3, True, True, 150),       # more images than SMs: several images per block
    (64, 0, 13, 3, 3, True, True, 210),       # the same for the compile-time 13x13 -> 5x5 geometry
])
@pytest.mark.parametrize("tc", ["tf32", "bf16"])
def test_permuted_conv_pool_tensor_core(tc, cout, out_sp, hw, k, R, anti, bias, D):
    from nesgpu_b200 import base
    from oracle import perturbed_ref as O
    from gpu_util import G, set_params
    cin = 32
    g = torch.Generator().manual_seed(cout + hw + D)
    layer = base.PermutedConv2d(cin, cout, k, D, bias=bias, antithetic=anti, permutation="out", out_sparsity=out_sp,
                                options={"tc": tc, "fuse": "relu_maxpool2"}).to(DEV)
    osp = layer.out_sparsity
    x = torch.randn(R * D, cin, hw, hw, generator=g)
    if tc == "bf16":
        x = x.bfloat16().float()          # the input arrives as bf16 in this mode: compare on representable values
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g) * .1 if bias else None
    eps = 0.05 * torch.randn(osp, cin, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g) if bias else None
    pout = torch.stack([torch.randperm(cout, generator=g) for _ in range(D)]).short()
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.output_permutations = G(eps), (G(beta) if bias else None), G(pout)
    want = O.permuted_conv2d_forward(x, W, b if bias else torch.zeros(cout), eps,
                                     beta if bias else torch.zeros(D, cout), None, pout, D, 1, 0, 1, anti)
    want = torch.nn.functional.max_pool2d(torch.relu(want), 2)
    before = C_launches()
    with torch.no_grad():
        layer.perturbed_flag = True
        y_nchw = layer.forward(G(x))                                                  # copies to channels-last first
        x_cl = G(x).contiguous(memory_format=torch.channels_last)
        y_cl = layer.forward(x_cl.bfloat16() if tc == "bf16" else x_cl)                # taken as is
    assert C_launches() - before == 4                                                 # 2 x (filter stack + fused kernel)
    assert _flag(_C()) == 0
    assert y_nchw.shape == want.shape and y_nchw.is_contiguous()
    assert rel_err(y_nchw, want) <= 2e-2 and rel_err(y_cl, want) <= 2e-2
    assert torch.equal(y_nchw, y_cl)
    # the perturbation itself is resolved: remove the member-independent part and compare what is left
    layer.weight_noise = G(torch.zeros_like(eps))
    with torch.no_grad():
        y0 = layer.forward(G(x))
    want0 = torch.nn.functional.max_pool2d(torch.relu(O.permuted_conv2d_forward(
        x, W, b if bias else torch.zeros(cout), torch.zeros_like(eps), beta if bias else torch.zeros(D, cout),
        None, pout, D, 1, 0, 1, anti)), 2)
    assert rel_err(y_nchw - y0, want - want0) <= 5e-2


def test_conv_pool_tc_rejects_uncovered_shapes():
    C = _C()
    x = torch.zeros(2, 14, 14, 32, device=DEV)
    w = torch.zeros(64, 32, 3, 3, device=DEV)
    y = torch.zeros(2, 64, 6, 6, device=DEV)
    buf = torch.zeros(1 << 18, dtype=torch.uint8, device=DEV)
    with pytest.raises(NotImplementedError):       # 12x12 outputs: pooled part needs more than 128 columns
        C.call("nes_permuted_conv_pool_fwd_tc", C.ptr(x), C.ptr(w), None, C.ptr(w), None, None, C.ptr(y), 2, 1,
               32, 14, 14, 64, 3, 3, 64, 0, C.ptr(buf), buf.numel(), C.stream())
    with pytest.raises(NotImplementedError):       # 16 input channels
        C.call("nes_permuted_conv_pool_fwd_tc", C.ptr(x), C.ptr(w), None, C.ptr(w), None, None, C.ptr(y), 2, 1,
               16, 13, 13, 64, 3, 3, 64, 0, C.ptr(buf), buf.numel(), C.stream())


@pytest.mark.parametrize("cout,out_sp,R,anti,bias,D", [
    (64, 0, 2, False, True, 6),
    (64, 0.5, 3, True, True, 4),
    (40, 0, 1, False, False, 2),
    (64, 0, 3, True, True, 210),          # more pairs than SMs
])
def test_permuted_conv_pool_two_images_per_mma(cout, out_sp, R, anti, bias, D):
    """bf16 fused kernel fed with the pair layout (images 2q and 2q+1 interleaved by pixel)."""
    from nesgpu_b200 import base
    from oracle import perturbed_ref as O
    from gpu_util import G, set_params
    cin, hw, k = 32, 13, 3
    g = torch.Generator().manual_seed(cout + D + R)
    layer = base.PermutedConv2d(cin, cout, k, D, bias=bias, antithetic=anti, permutation="out", out_sparsity=out_sp,
                                options={"tc": "bf16", "fuse": "relu_maxpool2", "in_layout": "bf16x2"}).to(DEV)
    osp = layer.out_sparsity
    x = torch.randn(R * D, cin, hw, hw, generator=g).bfloat16().float()
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g) * .1 if bias else None
    eps = 0.05 * torch.randn(osp, cin, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g) if bias else None
    pout = torch.stack([torch.randperm(cout, generator=g) for _ in range(D)]).short()
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.output_permutations = G(eps), (G(beta) if bias else None), G(pout)
    want = O.permuted_conv2d_forward(x, W, b if bias else torch.zeros(cout), eps,
                                     beta if bias else torch.zeros(D, cout), None, pout, D, 1, 0, 1, anti)
    want = torch.nn.functional.max_pool2d(torch.relu(want), 2)
    B = R * D
    xp = x.permute(0, 2, 3, 1).reshape(B // 2, 2, hw, hw, cin).permute(0, 2, 3, 1, 4).reshape(B // 2, hw, hw, 2 * cin)
    xp = G(xp).bfloat16().contiguous().permute(0, 3, 1, 2)             # (B/2, 64, 13, 13), channels-last
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(xp)
    assert _flag(_C()) == 0
    assert y.shape == want.shape
    assert rel_err(y, want) <= 2e-2
    with pytest.raises(NotImplementedError):                            # the layout is only readable by this kernel
        layer.options = dict(layer.options, tc="tf32")
        layer.forward(xp)


def test_pair_kernel_full_size_matches_single_image_kernel():
    """One forward chunk of the ES configuration (1024 members x 16 images): every block works through ~55 pairs, so
    the stage / accumulator / eps-buffer phases wrap many times.  The pair kernel and the one-image bf16 kernel do
    the same products; they differ only by the bf16 rounding of the noise rows the pair kernel stages."""
    from nesgpu_b200 import base
    D, R, cin, cout, hw = 1024, 16, 32, 64, 13
    g = torch.Generator().manual_seed(99)
    one = base.PermutedConv2d(cin, cout, 3, D, permutation="out", options={"tc": "bf16", "fuse": "relu_maxpool2"}).to(DEV)
    two = base.PermutedConv2d(cin, cout, 3, D, permutation="out",
                              options={"tc": "bf16", "fuse": "relu_maxpool2", "in_layout": "bf16x2"}).to(DEV)
    one.set_seed(5)
    one.set_noise(0.02)
    with torch.no_grad():
        two.weight.copy_(one.weight)
        two.bias.copy_(one.bias)
    two.weight_noise, two.bias_noise, two.output_permutations = one.weight_noise, one.bias_noise, one.output_permutations
    B = R * D
    x = torch.randn(B, hw, hw, cin, generator=g).bfloat16().to(DEV)                    # channels-last storage
    xp = x.view(B // 2, 2, hw, hw, cin).permute(0, 2, 3, 1, 4).reshape(B // 2, hw, hw, 2 * cin).contiguous()
    with torch.no_grad():
        one.perturbed_flag = two.perturbed_flag = True
        y1 = one.forward(x.permute(0, 3, 1, 2))
        y2 = two.forward(xp.permute(0, 3, 1, 2))
    assert _flag(_C()) == 0
    assert y1.shape == y2.shape == (B, cout, 5, 5)
    assert rel_err(y2, y1.cpu()) <= 1e-3
    # every image of every block was written (no stale rows): compare a few single images exactly in structure
    assert torch.isfinite(y2).all() and (y2 >= 0).all()


# ------------------------------------------------------------------ output-permuted PermutedLinear, one cluster kernel

def _perm_out_case(D, R, in_f, out_f, out_sp, seed, bias=True, beta=True, identity=False, antithetic=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(R * D, in_f, generator=g)
    W = torch.randn(out_f, in_f, generator=g) / in_f ** .5
    b = torch.randn(out_f, generator=g) if bias else None
    eps = 0.05 * torch.randn(out_sp, in_f, generator=g)
    bn = 0.02 * torch.randn(D, out_f, generator=g) if beta else None
    pout = None if identity else torch.stack([torch.randperm(out_f, generator=g) for _ in range(D)]).short()
    return x, W, b, eps, bn, pout


def _perm_out_run(C, case, D, R, mode, antithetic=True):
    x, W, b, eps, bn, pout = case
    in_f, out_f, out_sp = x.shape[1], W.shape[0], eps.shape[0]
    assert C.call("nes_permuted_linear_out_fwd_tc_supported", D, R, in_f, out_f, out_sp, mode) == 1
    y = torch.full((R * D, out_f), float("nan"), device=DEV)
    gx, gW, gb, ge, gbn, gp = G(x), G(W), G(b), G(eps), G(bn), G(pout)
    before = C.call("nes_launch_count")
    C.call("nes_permuted_linear_out_fwd_tc", C.ptr(gx), C.ptr(gW), C.ptr(gb), C.ptr(ge), C.ptr(gbn), C.ptr(gp), C.ptr(y),
           D, R, in_f, out_f, out_sp, 1 if antithetic else 0, mode, C.stream())
    launches = C.call("nes_launch_count") - before
    torch.cuda.synchronize()
    return y, launches


@pytest.mark.parametrize("D,R,in_f,out_f,out_sp", [
    (512, 2, 256, 256, 256),      # the 256x256 benchmark layer: four blocks per cluster, 64 + 64 columns each
    (48, 2, 200, 136, 136),       # K tail (200 = 6 * 32 + 8), ragged column slices
    (48, 2, 200, 136, 34),        # sparse noise rows: most gathers hit the zero rule
    (7, 3, 36, 10, 10),           # one partial row tile, a single block per cluster
    (300, 1, 64, 1000, 500),      # wide layer: eight blocks per cluster
    (1, 1, 4, 1, 1),
    (130, 2, 128, 48, 16),
])
def test_permuted_linear_out_cluster_kernel_vs_oracle(D, R, in_f, out_f, out_sp):
    from nesgpu_b200 import _cabi as C
    from oracle import perturbed_ref as O
    case = _perm_out_case(D, R, in_f, out_f, out_sp, seed=D + in_f + out_f)
    x, W, b, eps, bn, pout = case
    want = O.permuted_linear_forward(x, W, b, eps, bn, None, pout, D, True)
    base_only = x @ W.t() + b
    y3, launches = _perm_out_run(C, case, D, R, 3)
    assert launches == 1                                        # no pre-pass, no scratch: one kernel
    assert_close(y3, want, tol=1e-4, what="3xTF32")
    # the perturbation term on its own (it is what the ES update sees) within 1e-3
    assert_close(y3.cpu() - base_only, want - base_only, tol=1e-3, what="perturbation term")
    y1, _ = _perm_out_run(C, case, D, R, 1)
    assert_close(y1, want, tol=2e-2, what="TF32 (stated mode)")
    assert _flag(C) == 0


def test_permuted_linear_out_cluster_kernel_options():
    """No bias, no bias noise, identity output map (pout NULL), non-antithetic repeats."""
    from nesgpu_b200 import _cabi as C
    from oracle import perturbed_ref as O
    D, R, in_f, out_f = 40, 3, 96, 80
    for bias, beta, identity, anti in [(False, True, False, True), (True, False, False, False), (True, True, True, True),
                                       (False, False, True, False)]:
        case = _perm_out_case(D, R, in_f, out_f, out_f, seed=5, bias=bias, beta=beta, identity=identity)
        x, W, b, eps, bn, pout = case
        want = O.permuted_linear_forward(x, W, b, eps, bn, None, pout, D, anti)
        y, _ = _perm_out_run(C, case, D, R, 3, antithetic=anti)
        assert_close(y, want, tol=1e-4, what="bias=%s beta=%s identity=%s anti=%s" % (bias, beta, identity, anti))


def test_permuted_linear_out_cluster_kernel_refuses_uncovered_shapes():
    from nesgpu_b200 import _cabi as C
    assert C.call("nes_permuted_linear_out_fwd_tc_supported", 8, 1, 30, 16, 16, 3) == 0        # in % 4 != 0
    assert C.call("nes_permuted_linear_out_fwd_tc_supported", 8, 1, 32, 2000, 2000, 3) == 0    # out + out_sp > 2048
    assert C.call("nes_permuted_linear_out_fwd_tc_supported", 8, 1, 32, 16, 16, 2) == 0        # no bf16 form
    d = torch.zeros(64, device=DEV)
    with pytest.raises(NotImplementedError):
        C.call("nes_permuted_linear_out_fwd_tc", C.ptr(d), C.ptr(d), None, C.ptr(d), None, None, C.ptr(d),
               8, 1, 30, 16, 16, 0, 3, C.stream())


# ------------------------------------------------------------------ split-bf16 convolutions: the fp32 bar on the tensor cores

@pytest.mark.parametrize("mode,in_sp,out_sp,R,anti,hw,k,pad,cout,cin", [
    ("out", 0, 0.5, 1, False, 13, 3, 1, 64, 64), ("in", 0, 0, 2, True, 9, 3, 1, 32, 64), ("both", 0, 0, 3, True, 8, 3, 0, 64, 64),
    ("out", 0, 0, 2, True, 33, 1, 0, 128, 128), ("auto", 0.5, 0, 1, False, 20, 3, 2, 24, 64), ("out", 0, 0, 2, True, 32, 3, 1, 64, 64),
    # the form with the filter in tensor memory (64 input channels, <= 64 output channels, noise rows within 80 KB):
    # antithetic pairs over several tiles, a 1x1 filter with a ragged channel count and an odd repeat count
    ("out", 0, 0.25, 2, True, 32, 3, 1, 32, 64), ("out", 0, 0.5, 3, True, 10, 1, 0, 24, 64), ("out", 0, 0.125, 1, False, 17, 2, 1, 56, 64),
    # an image too large for the form with the filter in shared memory: only the tensor-memory form covers it
    ("out", 0, 0.5, 1, False, 64, 3, 1, 64, 64),
])
def test_permuted_conv_split_bf16_holds_the_fp32_bar(mode, in_sp, out_sp, R, anti, hw, k, pad, cout, cin):
    """Default mode of a covered geometry: three bf16 products on hi/lo splits; 1e-4 on the output and 1e-3 on the
    perturbation term alone (the part the ES update sees)."""
    from nesgpu_b200 import base, _cabi as C
    from oracle import perturbed_ref as O
    from gpu_util import set_params
    D = 5
    g = torch.Generator().manual_seed(hw + k + cout)
    layer = base.PermutedConv2d(cin, cout, k, D, padding=pad, antithetic=anti, permutation=mode, in_sparsity=in_sp,
                                out_sparsity=out_sp).to(DEV)
    isp, osp = layer.in_sparsity, layer.out_sparsity
    x = torch.randn(R * D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g)
    eps = 0.05 * torch.randn(osp, isp, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g)
    pin = _perms(g, D, cin, isp) if layer.permute_inputs else None
    pout = _perms(g, D, cout) if layer.permute_outputs else None
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(eps), G(beta)
    layer.input_permutations, layer.output_permutations = G(pin), G(pout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    torch.cuda.synchronize()
    assert layer.last_path == "bf16x3" and _flag(C) == 0
    want = O.permuted_conv2d_forward(x, W, b, eps, beta, pin, pout, D, 1, pad, 1, anti)
    assert_close(y, want, tol=1e-4, what="split-bf16 conv")
    basey = torch.nn.functional.conv2d(x, W, b, 1, pad)
    assert_close(y.cpu() - basey, want - basey, tol=1e-3, what="perturbation term")
    layer.options = {"tc": "fp32"}
    with torch.no_grad():
        y32 = layer.forward(G(x))
    assert layer.last_path == "fp32"
    assert_close(y32, want, tol=1e-4, what="CUDA-core conv")


def test_permuted_conv_split_bf16_many_members_per_block():
    """More members than SMs: a block builds several member filters in turn (the W tile ring runs across members)."""
    from nesgpu_b200 import base, _cabi as C
    from oracle import perturbed_ref as O
    from gpu_util import set_params
    D, cin, cout, hw, k = 333, 64, 64, 8, 3
    g = torch.Generator().manual_seed(77)
    layer = base.PermutedConv2d(cin, cout, k, D, padding=1, antithetic=False, permutation="out", out_sparsity=0.5).to(DEV)
    osp = layer.out_sparsity
    x = torch.randn(D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g)
    eps = 0.05 * torch.randn(osp, cin, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g)
    pout = _perms(g, D, cout)
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise = G(eps), G(beta)
    layer.output_permutations = G(pout)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    torch.cuda.synchronize()
    assert layer.last_path == "bf16x3" and _flag(C) == 0
    want = O.permuted_conv2d_forward(x, W, b, eps, beta, None, pout, D, 1, 1, 1, False)
    assert_close(y, want, tol=1e-4, what="split-bf16 conv, 333 members")
    basey = torch.nn.functional.conv2d(x, W, b, 1, 1)
    assert_close(y.cpu() - basey, want - basey, tol=1e-3, what="perturbation term")


def test_perturbed_conv_split_bf16_holds_the_fp32_bar():
    from nesgpu_b200 import base, _cabi as C
    from oracle import perturbed_ref as O
    from gpu_util import set_params
    D, R, cin, cout, hw, k = 4, 2, 64, 64, 12, 3
    g = torch.Generator().manual_seed(31)
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
    torch.cuda.synchronize()
    assert layer.last_path == "bf16x3" and _flag(C) == 0
    want = O.perturbed_conv2d_forward(x, W, b, E, beta, D, 1, 1, 1, True)
    assert_close(y, want, tol=1e-4, what="split-bf16 conv")
    basey = torch.nn.functional.conv2d(x, W, b, 1, 1)
    assert_close(y.cpu() - basey, want - basey, tol=1e-3, what="perturbation term")


def test_split_bf16_is_not_taken_for_uncovered_geometries():
    from nesgpu_b200 import base, _cabi as C
    assert C.call("nes_conv2d_fwd_bf16x3_supported", 64, 32, 32, 64, 3, 3, 1, 1, 1, 1, 1, 1) == 1
    assert C.call("nes_conv2d_fwd_bf16x3_supported", 32, 13, 13, 64, 3, 3, 1, 1, 0, 0, 1, 1) == 0      # 32 input channels
    assert C.call("nes_conv2d_fwd_bf16x3_supported", 64, 32, 32, 64, 3, 3, 2, 2, 1, 1, 1, 1) == 0      # stride 2
    layer = base.PermutedConv2d(64, 64, 3, 4, padding=1, options={"tc": "bf16x3"}, stride=2).to(DEV)
    layer.set_noise(0.02)
    layer.perturbed_flag = True
    with pytest.raises(NotImplementedError):
        layer.forward(torch.zeros(4, 64, 8, 8, device=DEV))


@pytest.mark.parametrize("cout,out_sp,hw,k,R,anti,bias,D", [
    (64, 0, 13, 3, 2, True, True, 5), (64, 0.5, 13, 3, 4, True, True, 3), (40, 0, 12, 3, 1, False, False, 7),
    (64, 0, 13, 3, 3, True, True, 210),
])
def test_permuted_conv_pool_split_bf16_holds_the_fp32_bar(cout, out_sp, hw, k, R, anti, bias, D):
    """Fused Conv + ReLU + MaxPool2d(2) in the three-product split-bf16 form: 1e-4 against the oracle on an fp32
    input (split into hi + lo bf16 parts on the way in), 1e-3 on the perturbation term alone."""
    from nesgpu_b200 import base
    from oracle import perturbed_ref as O
    from gpu_util import set_params
    cin = 32
    g = torch.Generator().manual_seed(cout + hw + D + 1)
    layer = base.PermutedConv2d(cin, cout, k, D, bias=bias, antithetic=anti, permutation="out", out_sparsity=out_sp,
                                options={"tc": "bf16x3", "fuse": "relu_maxpool2"}).to(DEV)
    osp = layer.out_sparsity
    x = torch.randn(R * D, cin, hw, hw, generator=g)
    W = torch.randn(cout, cin, k, k, generator=g) / (cin * k * k) ** .5
    b = torch.randn(cout, generator=g) * .1 if bias else None
    eps = 0.05 * torch.randn(osp, cin, k, k, generator=g)
    beta = 0.02 * torch.randn(D, cout, generator=g) if bias else None
    pout = torch.stack([torch.randperm(cout, generator=g) for _ in range(D)]).short()
    set_params(layer, W, b)
    layer.weight_noise, layer.bias_noise, layer.output_permutations = G(eps), (G(beta) if bias else None), G(pout)
    zb, zbeta = (b if bias else torch.zeros(cout)), (beta if bias else torch.zeros(D, cout))
    pre = O.permuted_conv2d_forward(x, W, zb, eps, zbeta, None, pout, D, 1, 0, 1, anti)
    want = torch.nn.functional.max_pool2d(torch.relu(pre), 2)
    with torch.no_grad():
        layer.perturbed_flag = True
        y = layer.forward(G(x))
    assert layer.last_path == "bf16x3" and _flag(_C()) == 0
    assert_close(y, want, tol=1e-4, what="split-bf16 fused layer")
    layer.weight_noise = G(torch.zeros_like(eps))
    with torch.no_grad():
        y0 = layer.forward(G(x))
    want0 = torch.nn.functional.max_pool2d(torch.relu(O.permuted_conv2d_forward(x, W, zb, torch.zeros_like(eps), zbeta, None, pout,
                                                                                D, 1, 0, 1, anti)), 2)
    assert_close(y - y0, want - want0, tol=1e-3, what="perturbation term")
