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


def assert_close(got, want, tol=REL_TOL, what=""):
    e = rel_err(got, want)
    assert e <= tol, "%s rel err %.3e > %.1e" % (what, e, tol)


def set_params(layer, weight, bias):
    with torch.no_grad():
        layer.weight.copy_(G(weight))
        if bias is not None:
            layer.bias.copy_(G(bias))
