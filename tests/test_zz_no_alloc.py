"""The allocation-free SSD entry point (`b200_mamba_chunk_scan_combined_static`).

Some callers cannot allocate device memory: a plugin that a host runtime hands nothing but its input and output tensors,
or code running where cudaMalloc is off limits. For them the library carries a fixed 64 MiB scratch array in its own
device image. This test drives that entry point through the C ABI twice in a row (the second call with other inputs and
another shape, so stale scratch contents from the first would show) and checks each result against the ordinary
entry point fed with a caller-provided workspace. Both run the same kernels on the same data, so the results must be
identical bit for bit; the assertion still states the f16 tolerance used elsewhere (rel 2e-2 / abs 2e-3) as the bound.
Each result of the static entry point is also compared with the CPU oracle directly (same rule, zero elements outside),
so that it does not stand on its sibling alone.

This file sorts last on purpose: a run that stops at the first failure has already executed every other test.
"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle as orc  # noqa: E402
from tolerance import assert_close_f16  # noqa: E402

pytestmark = pytest.mark.gpu


def _inputs(seed, b, l, H, P, G, N):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rn = lambda *s, std=1.0: (torch.randn(*s, device="cuda", generator=g) * std).half()
    x, dt, B, C = rn(b, l, H, P, std=0.5), rn(b, l, H), rn(b, l, G, N, std=0.5), rn(b, l, G, N, std=0.5)
    A = -(torch.rand(H, device="cuda", generator=g) * 15 + 1)
    D = torch.ones(H, device="cuda")
    dt_bias = torch.full((H,), -3.0, device="cuda")
    init = torch.randn(b, H, P, N, device="cuda", generator=g) * 0.1
    return x, dt, A, B, C, D, dt_bias, init


def _run(lib, capi, static, x, dt, A, B, C, D, dt_bias, init, chunk):
    b, l, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    y = torch.empty_like(x)
    fs = torch.empty(b, H, P, N, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    common = [capi.F16, p(x), H * P, p(dt), H, p(A), 0, p(B), G * N, p(C), G * N, p(D), p(dt_bias), p(init), p(y), H * P, p(fs),
              b, l, H, P, G, N, chunk, 1]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if static:
        capi.call("b200_mamba_chunk_scan_combined_static", *common, stream)
    else:
        nbytes = lib.b200_mamba_chunk_scan_combined_workspace_bytes(b, l, H, P, G, N, chunk)
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        capi.call("b200_mamba_chunk_scan_combined", *common, p(ws), nbytes, stream)
    torch.cuda.synchronize()
    return y.float().cpu().numpy(), fs.cpu().numpy()


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from anygpu_b200 import capi
    lib = capi.load()
    assert lib.b200_mamba_chunk_scan_combined_static_capacity() == 64 << 20
    # two calls in a row on the shared scratch: a tensor-core shape first, then a smaller SIMT-path shape
    for seed, dims, chunk in [(1, (2, 512, 8, 64, 1, 64), 256), (2, (1, 96, 4, 32, 2, 16), 32)]:
        args = _inputs(seed, *dims)
        y_ws, fs_ws = _run(lib, capi, False, *args, chunk)
        y_st, fs_st = _run(lib, capi, True, *args, chunk)
        assert np.isfinite(y_st).all() and np.abs(y_st).max() > 0
        assert_close_f16(y_st, y_ws, f"y, static vs workspace entry point {dims}")
        assert_close_f16(fs_st, fs_ws, f"final_states, static vs workspace entry point {dims}")
        assert np.array_equal(y_st, y_ws) and np.array_equal(fs_st, fs_ws)
        x, dt, A, B, C, D, dt_bias, init = (t.float().cpu().numpy() for t in args)
        wy, wfs = orc.ssd_chunk_scan(x, dt, A, B, C, chunk, D=D, dt_bias=dt_bias, initial_states=init)
        assert_close_f16(y_st, wy, f"y, static entry point vs oracle {dims}")
        assert_close_f16(fs_st, wfs, f"final_states, static entry point vs oracle {dims}")


def test_static_scratch_entry_point_rejects_oversized_problems():
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from anygpu_b200 import capi
    lib = capi.load()
    one = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    # batch 16 x 4096 tokens x 64 heads needs far more than 64 MiB of scratch
    assert lib.b200_mamba_chunk_scan_combined_workspace_bytes(16, 4096, 64, 64, 1, 64, 256) > (64 << 20)
    rc = lib.b200_mamba_chunk_scan_combined_static(capi.F16, one, 4096, one, 64, one, 0, one, 64, one, 64, None, None, None, one, 4096,
                                                   None, 16, 4096, 64, 64, 1, 64, 256, 1, None)
    assert rc == -3
    assert lib.b200_status_string(rc) == b"workspace missing or too small"
