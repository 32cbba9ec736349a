"""CPU-side checks of the boundary: the shared library loads, exports every symbol the header
declares, and the host-side layer logic follows the reference's constructor rules.  No compute
call is made (no GPU needed)."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "nesgpu_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nes_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from nesgpu_b200 import _cabi
    lib = ctypes.CDLL(_cabi.lib_path)
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), name
    # and the ctypes table covers exactly the declared entry points
    assert sorted(_cabi.SIGNATURES) == names


def test_status_strings_and_version():
    from nesgpu_b200 import _cabi
    assert _cabi.lib.nes_abi_version() == 1
    for code in (0, -1, -2, -3, -4, -5):
        assert _cabi.lib.nes_status_string(code)
    assert _cabi.lib.nes_status_string(-99) == b"unknown status"


def test_scratch_size_queries_are_pure():
    from nesgpu_b200 import _cabi
    L = _cabi.lib
    assert L.nes_perturbed_update_scratch_bytes(0, 100) == 0
    n = 1 << 20
    b = L.nes_perturbed_update_scratch_bytes(1024, n)
    assert b % (4 * n) == 0 and 0 <= b <= 16 * 4 * n
    assert L.nes_permuted_linear_fwd_scratch_bytes(512, 2, 256) == 512 * 2 * 256 * 4
    assert L.nes_permuted_conv2d_fwd_scratch_bytes(10, 3, 5) == 10 * 8 * 2
    assert L.nes_permuted_update_scratch_bytes(20, 10, 7, 10) == max(10 * 10, 7 * 20) * 4
    assert L.nes_bin_weighted_sum_scratch_bytes(1024, 1024, 16, 64) >= 1024 * 1024 * 4


def test_constructor_rule_matches_reference(perturbed_golden):
    from nesgpu_b200.base import PermutedLinear
    for rule in perturbed_golden.meta["__constructor_rules__"]:
        in_d, out_d, mode, isp, osp = rule["args"]
        layer = PermutedLinear(in_d, out_d, 2, permutation=mode, in_sparsity=isp, out_sparsity=osp)
        got = [layer.permute_inputs, layer.permute_outputs, layer.in_sparsity, layer.out_sparsity]
        assert got == rule["result"], rule


def test_layer_api_surface():
    import modules.base as mb
    from nesgpu_b200 import base
    for name in ["PerturbedModel", "Perturbed", "Permuted", "PerturbedLinear", "PerturbedConv2d",
                 "PermutedLinear", "PermutedConv2d", "SparsePerturbedLinear"]:
        assert getattr(mb, name) is getattr(base, name)
    for meth in ["set_noise_scale", "set_noise", "set_seed", "allocate_weight", "allocate_bias",
                 "allocate_memory", "free_memory", "weight_grad", "update"]:
        assert callable(getattr(base.Perturbed, meth))
    for meth in ["apply_input_permutation", "apply_output_permutation", "get_permutation_weights"]:
        assert callable(getattr(base.Permuted, meth))
    layer = base.PermutedConv2d(4, 8, 3, 16, padding=1, out_sparsity=.5)
    assert (layer.permute_inputs, layer.permute_outputs, layer.out_sparsity, layer.in_sparsity) == (False, True, 4, 4)
    assert layer.weight_noise is None and layer.input_permutations is None and layer.perturbed_flag is False
    with pytest.raises(NotImplementedError):
        base.PermutedLinear(4, 4, 2, permutation="sideways")
    with pytest.raises(NotImplementedError):
        base.PermutedLinear(4, 4, 2, permutation="both", options={"combined": True})


def test_population_wrapper_broadcasts():
    from nesgpu_b200 import base
    net = torch.nn.Sequential(base.PermutedLinear(6, 5, 4), torch.nn.ReLU(), base.PerturbedLinear(5, 3, 4))
    pm = base.PerturbedModel(net, 4)
    assert len(pm.perturbed_layers) == 2
    pm.set_noise_scale(0.5)
    pm.set_seed(7)
    assert all(l.noise_scale == 0.5 and l.seed == 7 for l in pm.perturbed_layers)
    seen = []
    net.probe = lambda: seen.append([l.perturbed_flag for l in pm.perturbed_layers]) or "ok"
    assert pm.probe() == "ok" and seen == [[True, True]]
    assert all(not l.perturbed_flag for l in pm.perturbed_layers)


def test_no_cpu_fallback():
    from nesgpu_b200 import base
    layer = base.PerturbedLinear(4, 3, 2)
    with pytest.raises(RuntimeError, match="CUDA"):
        layer.forward(torch.zeros(2, 4))
    import nesgpu_b200.boolean_operations as bo
    with pytest.raises(RuntimeError, match="CUDA"):
        bo.pack(torch.zeros(2, 64, dtype=torch.bool), torch.int64)
