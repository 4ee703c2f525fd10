"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol the header declares, and rejects
bad arguments with status codes before touching the GPU (no compute is launched here)."""
import ctypes
import os
import re

import pytest

from anygpu_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "b200_mamba2.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_list_the_same_functions():
    assert declared_functions() == sorted(capi.SIGNATURES)


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    for name in declared_functions():
        assert hasattr(lib, name), name
    assert lib.b200_abi_version() == 3
    assert lib.b200_status_string(0) == b"ok"
    assert lib.b200_status_string(-4) == b"device-side wait timed out"


def test_null_and_shape_validation_needs_no_gpu():
    lib = capi.load()
    one = ctypes.c_void_p(256)  # never dereferenced: validation fails first
    assert lib.b200_linear(capi.F16, None, 8, one, 0, one, 8, 1, 8, 8, None) == -7
    assert lib.b200_linear(capi.F16, one, 8, one, 0, one, 8, 1, 0, 8, None) == -1
    assert lib.b200_linear(capi.F16, one, 4, one, 0, one, 8, 1, 8, 8, None) == -1  # ldx < K
    assert lib.b200_linear(capi.F16, one, 8, one, 7, one, 8, 1, 8, 8, None) == -6  # unknown weight layout
    # shapes TMA cannot address (K % 8 != 0) are routed to the SIMT kernel, like every fp32 problem
    assert lib.b200_linear_kernel_name(capi.F16, 4, 12, 8) == b"gemm_simt_kernel<__half>"
    assert lib.b200_linear_kernel_name(capi.F32, 4, 16, 8) == b"gemm_simt_kernel<float>"
    assert lib.b200_linear_kernel_name(capi.F16, 8192, 2048, 8384) == b"gemm_f16_tcgen05_pair_kernel"
    assert lib.b200_linear_kernel_name(capi.F16, 64, 2560, 10448).startswith(b"gemm_f16_tcgen05_kernel")
    assert lib.b200_launch_count(1) >= 0 and lib.b200_launch_count(0) == 0
    assert lib.b200_causal_conv1d(capi.F16, one, one, one, one, 1, 8, 8, 5, None) == -1  # width > 4
    assert lib.b200_causal_conv1d(capi.F16, one, None, one, one, 1, 8, 8, 4, None) == -7
    assert lib.b200_causal_conv1d(7, one, one, one, one, 1, 8, 8, 4, None) == -6
    assert lib.b200_causal_conv1d(capi.F16, one, one, one, one, 0, 8, 8, 4, None) == 0  # empty batch is a no-op
    assert lib.b200_causal_conv1d_tokens(capi.F16, one, 4, one, one, one, 8, None, None, 1, 8, 8, 4, None) == -1  # stride < dims
    assert lib.b200_causal_conv1d_update(capi.F16, one, 8, None, one, one, one, 8, 1, 8, 4, None) == -7
    assert lib.b200_gated_rmsnorm(capi.F16, one, 8, one, 8, one, one, 8, 1, 8, 3, 1e-5, None) == -1  # group does not divide d
    assert lib.b200_gated_rmsnorm(capi.F16, one, 8, one, 8, one, one, 8, 0, 8, 8, 1e-5, None) == 0
    args = [capi.F16, one, 64, one, 8, one, 0, one, 16, one, 16, None, None, None, one, 64, None]
    assert lib.b200_mamba_chunk_scan_combined(*args, 1, 32, 8, 8, 1, 16, 512, 1, one, 1 << 20, None) == -6  # chunk > 256
    assert lib.b200_mamba_chunk_scan_combined(*args, 1, 32, 8, 8, 3, 16, 32, 1, one, 1 << 20, None) == -1  # H % G != 0
    assert lib.b200_mamba_chunk_scan_combined(*args, 1, 32, 8, 8, 1, 16, 32, 1, None, 0, None) == -3  # no workspace
    assert lib.b200_mamba_chunk_scan_combined(*args, 1, 32, 8, 8, 1, 16, 32, 1, one, 16, None) == -3  # workspace too small
    assert lib.b200_selective_state_update(capi.F16, None, one, 64, one, 8, one, 0, one, 16, one, 16, None, None, one, 64,
                                           1, 8, 8, 1, 16, 1, None) == -7
    # host-buffer entry point: flag bits it does not know are refused before anything else is looked at
    cfg, w = capi.Mamba2Config(), capi.Mamba2Weights()
    assert lib.b200_mamba2_mixer_prefill_host_ex(capi.F16, ctypes.byref(cfg), ctypes.byref(w), one, one, 1, 8, one, 1 << 20, None, 2) == -6
    assert lib.b200_mamba2_mixer_prefill_host_ex(capi.F16, ctypes.byref(cfg), ctypes.byref(w), None, one, 1, 8, one, 1 << 20, None, 1) == -7


def test_workspace_queries():
    lib = capi.load()
    n = lib.b200_mamba_chunk_scan_combined_workspace_bytes(4, 2048, 64, 64, 1, 64, 256)
    assert n == 3 * 4 * 64 * 2048 * 4 + 4 * 8 * 64 * 64 * 64 * (4 + 2)
    cfg = capi.Mamba2Config(2048, 4096, 64, 64, 64, 1, 4, 256, 0, 1e-5)
    T = 4 * 2048
    want = T * 8384 * 2 + T * 4224 * 2 + T * 4096 * 2 + n
    assert lib.b200_mamba2_mixer_prefill_workspace_bytes(ctypes.byref(cfg), capi.F16, 4, 2048) == want
    assert lib.b200_mamba2_mixer_prefill_host_workspace_bytes(ctypes.byref(cfg), capi.F16, 4, 2048) == want + 2 * T * 2048 * 2
    bad = capi.Mamba2Config(2048, 4096, 63, 64, 64, 1, 4, 256, 0, 1e-5)  # nheads * headdim != d_inner
    assert lib.b200_mamba2_mixer_prefill_workspace_bytes(ctypes.byref(bad), capi.F16, 4, 2048) == 0
    w = capi.Mamba2Weights()
    assert lib.b200_mamba2_mixer_prefill(capi.F16, ctypes.byref(cfg), ctypes.byref(w), ctypes.c_void_p(256), ctypes.c_void_p(256),
                                         1, 8, None, None, None, None, 0, None) == -7  # null weights
    assert lib.b200_mamba2_mixer_decode_workspace_bytes(ctypes.byref(cfg), capi.F16, 64) > 0
    # packed variable-length batches: the workspace is that of one sequence of all the tokens; offsets are validated on the host
    assert lib.b200_mamba2_mixer_prefill_varlen_workspace_bytes(ctypes.byref(cfg), capi.F16, T) == \
        lib.b200_mamba2_mixer_prefill_workspace_bytes(ctypes.byref(cfg), capi.F16, 1, T)
    full = capi.Mamba2Weights(*([ctypes.c_void_p(256)] * 8))
    one = ctypes.c_void_p(256)
    cu = lambda *v: (ctypes.c_int64 * len(v))(*v)  # noqa: E731
    call = lambda c, n: lib.b200_mamba2_mixer_prefill_varlen(capi.F16, ctypes.byref(cfg), ctypes.byref(full), one, one, c, n,  # noqa: E731
                                                             None, None, None, None, 0, None)
    assert call(None, 1) == -7
    assert call(cu(1, 5), 1) == -1  # does not start at 0
    assert call(cu(0, 5, 3), 2) == -1  # decreasing
    assert call(cu(0, 0, 0), 2) == 0  # only empty sequences, no states wanted: nothing to do
    assert call(cu(0, 5), 1) == -3  # tokens but no workspace
