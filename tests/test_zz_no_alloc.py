"""The workspace-free variant of the fitness-weighted noise sum, called through the C ABI.

``nes_perturbed_update_noalloc`` is for hosts that can pass inputs and outputs but own no
device allocator (a plug-in inside a runtime that owns all device memory, a step that runs
where device memory must not be created): its partial sums live in a 16 MiB workspace built
into the library instead of a caller-provided ``scratch`` buffer.  The test calls it twice in
a row with different inputs -- the workspace keeps the first call's contents, so a stale read
would show in the second result -- and compares each result with ``nes_perturbed_update`` on
the same inputs and with the CPU restatement of the reference's update (``weights @ noise`` plus
the l1 / l2 terms).  Both entry points run the same kernels with the same member split, so the
results must agree to rounding (they are in fact bit-identical); the bound used is the
relative 1e-4 of the other fp32 parity tests.  This file sorts last on purpose.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_TOL = 1e-4
MAX_FLOATS = 4194304      # NES_NOALLOC_SCRATCH_FLOATS in include/nesgpu_b200.h


def _with_scratch(C, noise, w, weight, l1, l2):
    D, n = noise.shape[0], noise[0].numel()
    out = torch.empty(n, device=noise.device)
    nbytes = C.call("nes_perturbed_update_scratch_bytes", D, n)
    buf = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=noise.device)
    C.call("nes_perturbed_update", C.ptr(noise), C.ptr(w), C.ptr(weight), C.ptr(out), D, n, l1, l2,
           C.ptr(buf), nbytes, C.stream())
    return out, nbytes


def _no_alloc(C, noise, w, weight, l1, l2):
    D, n = noise.shape[0], noise[0].numel()
    out = torch.empty(n, device=noise.device)
    C.call("nes_perturbed_update_noalloc", C.ptr(noise), C.ptr(w), C.ptr(weight), C.ptr(out), D, n, l1, l2,
           C.stream())
    return out


def test_no_alloc_matches_scratch_entry_point_twice_in_a_row():
    from nesgpu_b200 import _cabi as C
    from oracle import perturbed_ref as O
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(31)
    used_workspace = False
    for D, n in [(256, 64 * 1024), (512, 4096), (96, 1001)]:      # split / split / scalar (n % 4 != 0) path
        weight = torch.randn(n, generator=g).to(dev)
        results = []
        for call in range(2):
            noise = torch.randn(D, n, generator=g).to(dev)
            w = (torch.rand(D, generator=g) * 2 - 1).to(dev)
            want, nbytes = _with_scratch(C, noise, w, weight, 0.01, 0.02)
            got = _no_alloc(C, noise, w, weight, 0.01, 0.02)
            torch.cuda.synchronize()
            used_workspace |= nbytes > 0
            err = ((got - want).norm() / want.norm()).item()
            assert err <= REL_TOL, "D=%d n=%d call %d: rel err %g" % (D, n, call, err)
            ref, _ = O.perturbed_update(weight.cpu(), noise.cpu(), None, w.cpu(), l1=0.01, l2=0.02)
            err = ((got.cpu() - ref).norm() / ref.norm()).item()
            assert err <= REL_TOL, "D=%d n=%d call %d: rel err %g against the oracle" % (D, n, call, err)
            results.append(got)
        assert not torch.equal(results[0], results[1])             # the two calls really differed
    assert used_workspace, "no case exercised the built-in workspace"


def test_no_alloc_takes_noise_that_is_not_16_byte_aligned():
    """A noise view that starts 4 bytes into an allocation makes the kernels fall back from 128-bit to scalar
    loads, which changes the member split; the entry point must size its workspace check for that plan too."""
    from nesgpu_b200 import _cabi as C
    from oracle import perturbed_ref as O
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(32)
    D, n = 256, 64 * 1024
    flat = torch.randn(D * n + 1, generator=g).to(dev)
    noise = flat[1:].view(D, n)
    assert noise.data_ptr() % 16 == 4
    w = (torch.rand(D, generator=g) * 2 - 1).to(dev)
    for call in range(2):
        got = _no_alloc(C, noise, w, None, 0.0, 0.0)
        want, _ = _with_scratch(C, noise, w, None, 0.0, 0.0)
        torch.cuda.synchronize()
        ref, _ = O.perturbed_update(torch.zeros(n), noise.cpu(), None, w.cpu())
        assert ((got - want).norm() / want.norm()).item() <= REL_TOL
        assert ((got.cpu() - ref).norm() / ref.norm()).item() <= REL_TOL


def test_no_alloc_rejects_sizes_beyond_its_workspace():
    from nesgpu_b200 import _cabi as C
    dev = torch.device("cuda")
    D, n = 1024, 2 * 1024 * 1024 + 1024                             # two splits of n floats: > 4 Mi floats
    assert C.call("nes_perturbed_update_scratch_bytes", D, n) > 4 * MAX_FLOATS
    # the size check comes before any memory is touched, so tiny stand-in buffers are enough
    dummy = torch.zeros(16, device=dev)
    with pytest.raises(NotImplementedError, match="built-in"):
        C.call("nes_perturbed_update_noalloc", C.ptr(dummy), C.ptr(dummy), None, C.ptr(dummy), D, n, 0.0, 0.0,
               C.stream())
