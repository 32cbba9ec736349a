"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

DEV = "cuda"
# fp32 paths: relative error bound stated by the port's contract
REL_TOL = 1e-4


def T(a, dtype=None):
    if a is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t if dtype is None else t.to(dtype)


def G(a, dtype=None):
    t = a if isinstance(a, torch.Tensor) else T(a)
    if t is None:
        return None
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV).contiguous()


def rel_err(got, want):
    got = got.detach().float().cpu().double()
    want = (want if isinstance(want, torch.Tensor) else T(want)).double()
    assert got.shape == want.shape, (got.shape, want.shape)
    denom = want.norm().item()
    return (got - want).norm().item() / (denom if denom > 0 else 1.0)


# a single element may be off by at most this many times tol * rms(want): the norm ratio alone would not
# see one wrong value in a tensor of millions of elements
MAX_ABS_FACTOR = 20.0


def max_abs_err(got, want):
    got = got.detach().float().cpu().double()
    want = (want if isinstance(want, torch.Tensor) else T(want)).double()
    return (got - want).abs().max().item() if want.numel() else 0.0


def assert_close(got, want, tol=REL_TOL, what=""):
    """Two bounds: the Frobenius-norm ratio <= tol, and every element within MAX_ABS_FACTOR * tol * rms(want)."""
    e = rel_err(got, want)
    assert e <= tol, "%s rel err %.3e > %.1e" % (what, e, tol)
    w = (want if isinstance(want, torch.Tensor) else T(want)).double()
    if w.numel():
        rms = (w.norm().item() / w.numel() ** .5) or 1.0
        worst = max_abs_err(got, want)
        bound = MAX_ABS_FACTOR * tol * rms
        assert worst <= bound, "%s max abs err %.3e > %.3e (rms %.3e)" % (what, worst, bound, rms)


def set_params(layer, weight, bias):
    with torch.no_grad():
        layer.weight.copy_(G(weight))
        if bias is not None:
            layer.bias.copy_(G(bias))
