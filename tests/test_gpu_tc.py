"""Tensor-core (tcgen05 / TMA) GEMM against a float64 CPU product.

Tolerances: mode 3 (3xTF32, error-compensated) must hold the fp32 bar (rel err <= 1e-4; it measures
~1e-6); mode 1 (plain TF32) is the stated reduced-precision mode with the 2e-2 bar (it measures ~5e-4)."""
import pytest
import torch

from gpu_util import DEV, rel_err

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
