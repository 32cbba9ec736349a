"""ctypes binding of ``libnesgpu_b200.so`` (the C ABI declared in ``include/nesgpu_b200.h``).

The library is the only compute path: if it is missing or fails to load, importing this
module raises -- there is no PyTorch or CPU fallback.  PyTorch is used for device memory,
streams and (elsewhere) process groups only.
"""
import ctypes
import os

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libnesgpu_b200.so")

c_i64, c_int, c_f32, c_u64, c_ptr = (ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_uint64,
                                     ctypes.c_void_p)

# name -> argument ctypes (return type is int unless listed in _RETURNS)
SIGNATURES = {
    "nes_abi_version": [],
    "nes_status_string": [c_int],
    "nes_last_error": [],
    "nes_launch_count": [],
    "nes_linear_fwd": [c_ptr] * 4 + [c_i64] * 3 + [c_ptr],
    "nes_linear_fwd_tc_scratch_bytes": [c_i64, c_i64, c_i64, c_int],
    "nes_linear_fwd_tc": [c_ptr] * 4 + [c_i64] * 3 + [c_int, c_ptr, c_i64, c_ptr],
    "nes_tc_error_flag": [c_ptr],
    "nes_conv2d_fwd": [c_ptr] * 4 + [c_i64] + [c_int] * 12 + [c_ptr],
    "nes_perturbed_linear_fwd": [c_ptr] * 6 + [c_i64] * 4 + [c_int] * 2 + [c_ptr],
    "nes_perturbed_conv2d_fwd": [c_ptr] * 6 + [c_i64] * 2 + [c_int] * 12 + [c_int, c_ptr],
    "nes_perturbed_update_scratch_bytes": [c_i64, c_i64],
    "nes_perturbed_update": [c_ptr] * 4 + [c_i64, c_i64, c_f32, c_f32, c_ptr, c_i64, c_ptr],
    "nes_perturbed_update_columns": [c_ptr] * 4 + [c_i64, c_i64, c_i64, c_f32, c_f32, c_ptr, c_i64, c_ptr],
    "nes_perturbed_update_direct": [c_ptr] * 5 + [c_i64, c_i64, c_f32, c_f32, c_ptr, c_i64, c_ptr],
    "nes_perturbed_update_noalloc": [c_ptr] * 4 + [c_i64, c_i64, c_f32, c_f32, c_ptr],
    "nes_sparse_perturbed_linear_fwd": [c_ptr] * 7 + [c_i64] * 4 + [c_int, c_int, c_ptr],
    "nes_sparse_perturbed_update": [c_ptr] * 5 + [c_i64] * 3 + [c_int, c_f32, c_f32, c_ptr],
    "nes_permuted_linear_fwd_scratch_bytes": [c_i64] * 3,
    "nes_permuted_linear_fwd": [c_ptr] * 8 + [c_i64] * 6 + [c_int, c_ptr, c_i64, c_ptr],
    "nes_permuted_linear_fwd_tc_scratch_bytes": [c_i64] * 5 + [c_int],
    "nes_permuted_linear_fwd_tc": [c_ptr] * 7 + [c_i64] * 6 + [c_int, c_int, c_ptr, c_i64, c_ptr],
    "nes_permuted_linear_out_fwd_tc_supported": [c_i64] * 5 + [c_int],
    "nes_permuted_linear_out_fwd_tc": [c_ptr] * 7 + [c_i64] * 5 + [c_int, c_int, c_ptr],
    "nes_shared_conv_pool_fwd": [c_ptr] * 5 + [c_i64, c_i64] + [c_int] * 6 + [c_ptr],
    "nes_permuted_conv_pool_fwd_tc_scratch_bytes": [c_int, c_int],
    "nes_permuted_conv_pool_fwd_tc": [c_ptr] * 7 + [c_i64, c_i64] + [c_int] * 8 + [c_ptr, c_i64, c_ptr],
    "nes_permuted_conv_pool_fwd_bf16": [c_ptr] * 7 + [c_i64, c_i64] + [c_int] * 8 + [c_ptr, c_i64, c_ptr],
    "nes_permuted_conv_pool_fwd_bf16x3_scratch_bytes": [c_int, c_int],
    "nes_permuted_conv_pool_fwd_bf16x3": [c_ptr] * 8 + [c_i64, c_i64] + [c_int] * 8 + [c_ptr, c_i64, c_ptr],
    "nes_permuted_conv_pool_fwd_bf16x2": [c_ptr] * 7 + [c_i64, c_i64] + [c_int] * 8 + [c_ptr, c_i64, c_ptr],
    "nes_permuted_conv2d_fwd_scratch_bytes": [c_i64, c_int, c_int],
    "nes_permuted_conv2d_fwd": [c_ptr] * 8 + [c_i64] * 2 + [c_int] * 12 + [c_int] * 3 + [c_ptr, c_i64, c_ptr],
    "nes_conv2d_fwd_tc_scratch_bytes": [c_i64, c_i64] + [c_int] * 8,
    "nes_perturbed_conv2d_fwd_tc": [c_ptr] * 6 + [c_i64] * 2 + [c_int] * 12 + [c_int, c_ptr, c_i64, c_ptr],
    "nes_permuted_conv2d_fwd_tc": [c_ptr] * 8 + [c_i64] * 2 + [c_int] * 12 + [c_int] * 3 + [c_ptr, c_i64, c_ptr],
    "nes_conv2d_fwd_bf16_scratch_bytes": [c_i64, c_i64] + [c_int] * 8,
    "nes_perturbed_conv2d_fwd_bf16": [c_ptr] * 6 + [c_i64] * 2 + [c_int] * 12 + [c_int, c_ptr, c_i64, c_ptr],
    "nes_permuted_conv2d_fwd_bf16": [c_ptr] * 8 + [c_i64] * 2 + [c_int] * 12 + [c_int] * 3 + [c_ptr, c_i64, c_ptr],
    "nes_conv2d_fwd_bf16x3_supported": [c_int] * 12,
    "nes_permuted_conv2d_fwd_bf16x3_supported": [c_int] * 15,
    "nes_conv2d_fwd_bf16x3_scratch_bytes": [c_i64, c_i64] + [c_int] * 8,
    "nes_perturbed_conv2d_fwd_bf16x3": [c_ptr] * 6 + [c_i64] * 2 + [c_int] * 12 + [c_int, c_ptr, c_i64, c_ptr],
    "nes_permuted_conv2d_fwd_bf16x3": [c_ptr] * 8 + [c_i64] * 2 + [c_int] * 12 + [c_int] * 3 + [c_ptr, c_i64, c_ptr],
    "nes_permuted_dense_noise": [c_ptr] * 4 + [c_i64] + [c_int] * 5 + [c_ptr],
    "nes_permuted_update_out": [c_ptr] * 7 + [c_i64] + [c_int] * 4 + [c_f32, c_f32, c_ptr],
    "nes_permuted_update_scratch_bytes": [c_int] * 4,
    "nes_permuted_update": [c_ptr] * 7 + [c_i64] + [c_int] * 5 + [c_f32, c_f32, c_ptr, c_i64, c_ptr],
    "nes_affine_fwd": [c_ptr] * 4 + [c_i64, c_i64, c_ptr],
    "nes_synthetic_linear_fwd_scratch_bytes": [c_i64] * 3,
    "nes_synthetic_linear_fwd": [c_ptr] * 8 + [c_i64] * 4 + [c_int, c_ptr, c_i64, c_ptr],
    "nes_synthetic_linear_fwd_tc_scratch_bytes": [c_i64] * 4 + [c_int],
    "nes_synthetic_linear_fwd_tc": [c_ptr] * 8 + [c_i64] * 4 + [c_int, c_int, c_ptr, c_i64, c_ptr],
    "nes_sparse_noise_add": [c_ptr] * 5 + [c_i64] * 4 + [c_int, c_int, c_ptr],
    "nes_synthetic_conv2d_fwd": [c_ptr] * 8 + [c_i64] * 2 + [c_int] * 12 + [c_int, c_ptr],
    "nes_synthetic_update_scratch_bytes": [c_int, c_int],
    "nes_synthetic_update": [c_ptr] * 6 + [c_i64] + [c_int] * 3 + [c_f32, c_f32, c_ptr, c_i64, c_ptr],
    "nes_fill_signs": [c_ptr, c_i64, c_u64, c_u64, c_ptr],
    "nes_fill_normal": [c_ptr, c_i64, c_f32, c_f32, c_u64, c_u64, c_ptr],
    "nes_fill_uniform": [c_ptr, c_i64, c_f32, c_f32, c_u64, c_u64, c_ptr],
    "nes_sample_permutations": [c_ptr, c_i64, c_int, c_int, c_int, c_u64, c_i64, c_ptr],
    "nes_bin_pack": [c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr],
    "nes_bin_int8pack": [c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr],
    "nes_bin_pack8": [c_ptr, c_ptr, c_i64, c_i64, c_ptr],
    "nes_bin_unpack": [c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr],
    "nes_bin_sample_bits": [c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_int, c_u64, c_ptr],
    "nes_bin_seeded_bmv": [c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_int, c_u64, c_ptr],
    "nes_bin_bmm": [c_ptr] * 3 + [c_i64] * 4 + [c_int, c_ptr],
    "nes_bin_bmm_act": [c_ptr] * 4 + [c_i64] * 4 + [c_int, c_ptr],
    "nes_bin_im2col": [c_ptr, c_ptr, c_i64] + [c_int] * 10 + [c_ptr],
    "nes_bin_conv": [c_ptr] * 5 + [c_i64] + [c_int] * 11 + [c_ptr],
    "nes_bin_weighted_sum_scratch_bytes": [c_i64, c_i64, c_i64, c_int],
    "nes_bin_weighted_sum": [c_ptr] * 3 + [c_i64] * 4 + [c_int, c_ptr, c_i64, c_ptr],
    "nes_bin_maxpool2d": [c_ptr, c_ptr, c_i64] + [c_int] * 10 + [c_ptr],
    "nes_binarized_probabilities": [c_ptr, c_ptr, c_ptr, c_i64, c_ptr],
    "nes_binarized_bias_noise": [c_ptr, c_i64, c_u64, c_u64, c_ptr],
    "nes_binarized_update_scratch_bytes": [c_i64, c_i64, c_i64, c_int],
    "nes_binarized_update": [c_ptr] * 6 + [c_i64] * 5 + [c_int, c_f32, c_f32, c_ptr, c_i64, c_ptr],
    "nes_binarized_linear_fwd_scratch_bytes": [c_i64, c_i64, c_int],
    "nes_binarized_linear_fwd": [c_ptr] * 5 + [c_i64] * 3 + [c_int] * 4 + [c_ptr, c_i64, c_ptr],
    "nes_binarized_conv_epilogue": [c_ptr] * 4 + [c_i64] * 3 + [c_int] * 4 + [c_ptr, c_ptr],
    "nes_binarized_int_threshold": [c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_int, c_ptr],
}
_RETURNS = {
    "nes_status_string": ctypes.c_char_p,
    "nes_last_error": ctypes.c_char_p,
    "nes_launch_count": c_i64,
    "nes_perturbed_update_scratch_bytes": c_i64,
    "nes_linear_fwd_tc_scratch_bytes": c_i64,
    "nes_synthetic_linear_fwd_scratch_bytes": c_i64,
    "nes_synthetic_linear_fwd_tc_scratch_bytes": c_i64,
    "nes_synthetic_update_scratch_bytes": c_i64,
    "nes_conv2d_fwd_tc_scratch_bytes": c_i64,
    "nes_conv2d_fwd_bf16_scratch_bytes": c_i64,
    "nes_permuted_linear_fwd_scratch_bytes": c_i64,
    "nes_permuted_linear_fwd_tc_scratch_bytes": c_i64,
    "nes_permuted_conv_pool_fwd_tc_scratch_bytes": c_i64,
    "nes_permuted_conv_pool_fwd_bf16x3_scratch_bytes": c_i64,
    "nes_permuted_conv2d_fwd_scratch_bytes": c_i64,
    "nes_permuted_update_scratch_bytes": c_i64,
    "nes_bin_weighted_sum_scratch_bytes": c_i64,
    "nes_permuted_linear_out_fwd_tc_supported": c_int,
    "nes_conv2d_fwd_bf16x3_supported": c_int,
    "nes_permuted_conv2d_fwd_bf16x3_supported": c_int,
    "nes_conv2d_fwd_bf16x3_scratch_bytes": c_i64,
    "nes_binarized_update_scratch_bytes": c_i64,
    "nes_binarized_linear_fwd_scratch_bytes": c_i64,
}
_NO_STATUS = set(_RETURNS) | {"nes_abi_version"}


def _load():
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            "nesgpu_b200: %s not found. Build it with `python -m nesgpu_b200.build`; there is no "
            "fallback path." % _LIB_PATH)
    lib = ctypes.CDLL(_LIB_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError if the library lacks a declared symbol
        fn.argtypes = args
        fn.restype = _RETURNS.get(name, c_int)
    if lib.nes_abi_version() != 1:
        raise RuntimeError("nesgpu_b200: ABI version mismatch")
    return lib


lib = _load()
lib_path = _LIB_PATH


class NesError(RuntimeError):
    pass


def call(name, *args):
    """Call an entry point that returns a status; raise NesError on failure."""
    rc = getattr(lib, name)(*args)
    if name in _NO_STATUS:
        return rc
    if rc != 0:
        detail = lib.nes_last_error().decode()
        what = lib.nes_status_string(rc).decode()
        if rc == -2:
            raise NotImplementedError("%s: %s (%s)" % (name, what, detail))
        raise NesError("%s: %s (%s)" % (name, what, detail))
    return rc


def check_device_errors():
    """Raise if a tensor-core kernel gave up on one of its bounded waits since the last check.

    Reading the device words synchronises the host with the device, so call this where the host waits
    anyway (after a step's results have been read); the words are cleared by the read."""
    flag = ctypes.c_int(0)
    call("nes_tc_error_flag", ctypes.byref(flag))
    if flag.value:
        role = {1: "TMA producer", 2: "MMA issuer", 3: "epilogue", 4: "filter builder / operand splitter"}
        raise NesError("a tensor-core kernel timed out in its %s wait (code %d); the outputs of that launch "
                       "are undefined" % (role.get(flag.value, "?"), flag.value))


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream():
    """The current CUDA stream of the current device, read at call time."""
    return torch.cuda.current_stream().cuda_stream


def require_cuda(t, name, dtype=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError("nesgpu_b200: %s must be a CUDA tensor (there is no CPU path)" % name)
    if dtype is not None and t.dtype != dtype:
        raise NotImplementedError("nesgpu_b200: %s must have dtype %s, got %s" % (name, dtype, t.dtype))
    return t if t.is_contiguous() else t.contiguous()


_scratch = {}


def scratch(nbytes, device):
    """A reusable byte buffer per (device, stream), grown on demand.  Kernels that use it
    are ordered by the stream, so reuse between consecutive calls is safe."""
    if nbytes <= 0:
        return None
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream())
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf
