"""GPU parity tests of the individual operators: every call goes through the C ABI (anygpu_b200.ops -> ctypes ->
libanygpu_b200.so) and is compared with the CPU oracle on identical seeded inputs, and with the golden vectors
generated from the anyGPU reference.

Tolerances: fp32 ops use the reference's own absolute rule 1e-3 (tests/test_tools.hpp:24-43) or tighter; f16 ops
use rel 2e-2 / abs 2e-3 (element passes if either holds) with ZERO elements allowed outside."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle as orc  # noqa: E402
from tolerance import assert_abs, assert_close_f16, rel_l2  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from anygpu_b200 import ops as _ops
    return _ops


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dtype)


def host(t):
    return t.float().cpu().numpy()


def f16v(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


def load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name + ".npz"))


# ---- causal conv1d --------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["conv1d_w4", "conv1d_w3", "conv1d_short"])
def test_conv1d_f32_golden(ops, golden_dir, name):
    g = load(golden_dir, name)
    y = host(ops.tensor_causal_conv1d(dev(g["x"]), dev(g["w"]), dev(g["b"])))
    # the reference checks CPU and CUDA against this golden at abs 1e-3 (tests/ext_torch_tests.cpp:745-778)
    assert_abs(y, g["y_torch"], name + " vs torch golden", 1e-3)
    assert_abs(y, g["y_ref"], name + " vs reference CPU", 1e-5)


@pytest.mark.parametrize("shape", [(2, 40, 64, 4), (1, 24, 128, 4), (3, 7, 19, 4), (2, 16, 8, 2), (1, 8, 4096, 4), (2, 5, 1, 4)])
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_conv1d_seq_layout(ops, shape, dtype):
    b, d, s, w = shape
    r = np.random.default_rng(b * 1000 + d + s)
    x, wt, bs = r.standard_normal((b, d, s), np.float32), r.standard_normal((d, w), np.float32) * 0.5, r.standard_normal(d).astype(np.float32) * 0.1
    if dtype == "f16":
        x, wt, bs = f16v(x), f16v(wt), f16v(bs)
        y = host(ops.tensor_causal_conv1d(dev(x, torch.float16), dev(wt, torch.float16), dev(bs, torch.float16)))
        assert_close_f16(y, orc.causal_conv1d(x, wt, bs), f"conv1d {shape}")
    else:
        y = host(ops.tensor_causal_conv1d(dev(x), dev(wt), dev(bs)))
        assert_abs(y, orc.causal_conv1d(x, wt, bs), f"conv1d {shape}", 1e-5)


@pytest.mark.parametrize("dims,stride,off", [(64, 200, 72), (24, 24, 0), (20, 52, 12), (528, 1064, 512)])
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_conv1d_token_layout_strided_with_states(ops, dims, stride, off, dtype):
    r = np.random.default_rng(dims)
    b, l, w = 2, 37, 4
    wide = r.standard_normal((b, l, stride), np.float32)
    wt, bs = r.standard_normal((dims, w), np.float32) * 0.5, r.standard_normal(dims).astype(np.float32) * 0.1
    init = r.standard_normal((b, dims, w - 1), np.float32)
    td = torch.float16 if dtype == "f16" else torch.float32
    if dtype == "f16":
        wide, wt, bs, init = map(f16v, (wide, wt, bs, init))
    x = wide[:, :, off:off + dims]
    # oracle: prepend the initial state as history, run the (b,c,l) operator, drop the history columns
    hist = np.concatenate([init, x.transpose(0, 2, 1)], axis=2)
    want = orc.causal_conv1d(hist, wt, bs)[:, :, w - 1:].transpose(0, 2, 1)
    wd = dev(wide, td)
    y, fin = ops.tensor_causal_conv1d_tokens(wd[:, :, off:off + dims], dev(wt, td), dev(bs, td), initial_state=dev(init, td),
                                             want_final_state=True)
    if dtype == "f16":
        assert_close_f16(host(y), want, "conv tokens")
    else:
        assert_abs(host(y), want, "conv tokens", 1e-5)
    assert np.array_equal(host(fin), hist[:, :, -(w - 1):])
    # without an initial state the left padding is zero
    y0 = ops.tensor_causal_conv1d_tokens(wd[:, :, off:off + dims], dev(wt, td), dev(bs, td))
    want0 = orc.causal_conv1d(np.ascontiguousarray(x.transpose(0, 2, 1)), wt, bs).transpose(0, 2, 1)
    (assert_close_f16 if dtype == "f16" else assert_abs)(host(y0), want0, "conv tokens zero pad")


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_conv1d_token_layout_weight_and_bias_views_off_the_vector_grid(ops, dtype):
    """Weights and biases that are views into larger buffers at an element offset that is not a multiple of 4: the vectorised
    body (one access per channel's 4 taps, one per 4 biases) cannot take them; the call must still give the oracle's result."""
    r = np.random.default_rng(23)
    b, l, dims, w = 2, 40, 64, 4
    td = torch.float16 if dtype == "f16" else torch.float32
    x = r.standard_normal((b, l, dims), np.float32)
    wt, bs = r.standard_normal((dims, w), np.float32) * 0.5, r.standard_normal(dims).astype(np.float32) * 0.1
    if dtype == "f16":
        x, wt, bs = map(f16v, (x, wt, bs))
    want = orc.causal_conv1d(np.ascontiguousarray(x.transpose(0, 2, 1)), wt, bs).transpose(0, 2, 1)
    for w_off, b_off in ((1, 0), (0, 3), (2, 1)):
        wbuf = torch.zeros(dims * w + 8, dtype=td, device="cuda")
        bbuf = torch.zeros(dims + 8, dtype=td, device="cuda")
        wv = wbuf[w_off:w_off + dims * w].view(dims, w)
        bv = bbuf[b_off:b_off + dims]
        wv.copy_(dev(wt, td))
        bv.copy_(dev(bs, td))
        y, fin = ops.tensor_causal_conv1d_tokens(dev(x, td), wv, bv, want_final_state=True)
        (assert_close_f16 if dtype == "f16" else assert_abs)(host(y), want, f"conv tokens, weight offset {w_off}, bias offset {b_off}")
        assert np.array_equal(host(fin), x[:, -(w - 1):].transpose(0, 2, 1))


def test_conv1d_short_sequence_final_state(ops):
    r = np.random.default_rng(5)
    x = f16v(r.standard_normal((2, 2, 16), np.float32))  # seqlen 2 < width-1
    wt, bs = f16v(r.standard_normal((16, 4), np.float32)), f16v(r.standard_normal(16).astype(np.float32))
    _, fin = ops.tensor_causal_conv1d_tokens(dev(x, torch.float16), dev(wt, torch.float16), dev(bs, torch.float16), want_final_state=True)
    want = np.concatenate([np.zeros((2, 16, 1), np.float32), x.transpose(0, 2, 1)], axis=2)
    assert np.array_equal(host(fin), want)


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_conv1d_update_reproduces_prefill(ops, dtype):
    r = np.random.default_rng(11)
    b, d, s, w = 3, 136, 24, 4
    x, wt, bs = r.standard_normal((b, d, s), np.float32), r.standard_normal((d, w), np.float32) * 0.5, r.standard_normal(d).astype(np.float32) * 0.1
    td = torch.float16 if dtype == "f16" else torch.float32
    if dtype == "f16":
        x, wt, bs = map(f16v, (x, wt, bs))
    full = orc.causal_conv1d(x, wt, bs)
    state = torch.zeros((b, d, w - 1), dtype=td, device="cuda")
    wd, bd = dev(wt, td), dev(bs, td)
    cols = [host(ops.tensor_causal_conv1d_update(dev(x[:, :, t], td), state, wd, bd)) for t in range(s)]
    got = np.stack(cols, axis=2)
    (assert_close_f16 if dtype == "f16" else assert_abs)(got, full, "conv update")
    assert np.array_equal(host(state), x[:, :, -(w - 1):])


# ---- gated RMSNorm ----------------------------------------------------------------------------------------------

def test_gated_rmsnorm_f32_golden(ops, golden_dir):
    g = load(golden_dir, "gated_rmsnorm")
    y = host(ops.tensor_zamba_gated_rmsnorm(dev(g["x"]), dev(g["z"]), dev(g["w"]), 4096, float(g["eps"])))
    # reference tolerance for this op: abs 1e-3 (tests/zamba2_tests.cpp:458-489)
    assert_abs(y, g["y_ref"], "vs reference CPU", 1e-4)
    assert_abs(y, g["y_torch"], "vs torch golden", 1e-4)


@pytest.mark.parametrize("rows,d,gsize", [(5, 4096, 4096), (3, 7168, 3584), (4, 512, 512), (2, 16384, 16384), (3, 100, 100), (2, 96, 24)])
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_gated_rmsnorm_shapes(ops, rows, d, gsize, dtype):
    r = np.random.default_rng(d + rows)
    x, z, w = r.standard_normal((rows, d), np.float32), r.standard_normal((rows, d), np.float32), r.standard_normal(d).astype(np.float32)
    td = torch.float16 if dtype == "f16" else torch.float32
    if dtype == "f16":
        x, z, w = map(f16v, (x, z, w))
    y = host(ops.tensor_zamba_gated_rmsnorm(dev(x, td), dev(z, td), dev(w, td), gsize, 1e-5, honor_gsize=True))
    want = orc.gated_rmsnorm(x, z, w, 1e-5, gsize=gsize)
    if dtype == "f16":
        assert_close_f16(y, want, "gated rmsnorm")
    else:
        assert_abs(y, want, "gated rmsnorm", 1e-4)


def test_gated_rmsnorm_ignores_gsize_like_the_reference(ops):
    r = np.random.default_rng(2)
    x, z, w = (r.standard_normal((4, 64), np.float32) for _ in range(3))
    w = w[0].copy()
    y = host(ops.tensor_zamba_gated_rmsnorm(dev(x), dev(z), dev(w), 16, 1e-5))
    assert_abs(y, orc.gated_rmsnorm(x, z, w, 1e-5), "whole-row statistic", 1e-5)


def test_gated_rmsnorm_strided_z(ops):
    r = np.random.default_rng(3)
    wide = f16v(r.standard_normal((6, 1064), np.float32))
    x, w = f16v(r.standard_normal((6, 512), np.float32)), f16v(r.standard_normal(512).astype(np.float32))
    wd = dev(wide, torch.float16)
    y = host(ops.tensor_zamba_gated_rmsnorm(dev(x, torch.float16), wd[:, :512], dev(w, torch.float16), 512, 1e-5))
    assert_close_f16(y, orc.gated_rmsnorm(x, wide[:, :512], w, 1e-5), "strided z")


# ---- linear -------------------------------------------------------------------------------------------------------

def test_linear_f32_golden(ops, golden_dir):
    g = load(golden_dir, "linear")
    y = host(ops.tensor_linear(dev(g["x"]), dev(g["w"])))
    # reference rule for fp32 linear: abs 1e-3 (tests/ext_torch_tests.cpp:519-552)
    assert_abs(y, g["y_ref"], "linear f32", 1e-4)


@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (128, 256, 256), (256, 512, 512), (64, 2560, 1064), (200, 264, 1064),
                                   (8, 64, 8), (300, 72, 520), (1024, 2048, 8384),
                                   (2304, 264, 2056), (2200, 512, 2312), (4096, 4096, 2048)])
@pytest.mark.parametrize("layout", ["KN", "NK"])
def test_linear_f16_tcgen05(ops, M, K, N, layout):
    r = np.random.default_rng(M + K + N)
    x = f16v(r.standard_normal((M, K), np.float32))
    w = f16v(r.standard_normal((K, N), np.float32) * 0.05)
    xd = dev(x, torch.float16)
    if layout == "KN":
        y = ops.tensor_linear(xd, dev(w, torch.float16))
    else:
        y = ops.tensor_linear(xd, dev(w.T.copy(), torch.float16), w_layout=ops.W_NK)
    torch.cuda.synchronize()
    from anygpu_b200 import capi
    assert capi.load().b200_last_device_error(None, None) == 0
    want = x.astype(np.float64) @ w.astype(np.float64)
    if M * K * N <= 64 * 2560 * 1064:
        want32 = orc.linear(x, w)  # the reference's accumulation order, fp32
        assert_abs(want32, want.astype(np.float32), "oracle self-check", 1e-2)
    assert_close_f16(host(y), want.astype(np.float32), f"linear f16 {M}x{K}x{N} {layout}")
    assert rel_l2(host(y), want) < 1e-3  # the reference's f16 mm test allows 1e-2 (tests/tests.cpp:138-165)


@pytest.mark.parametrize("M,K,N", [(33, 256, 644), (7, 100, 24), (130, 515, 515), (64, 256, 1064 + 4)])
@pytest.mark.parametrize("layout", ["KN", "NK"])
def test_linear_f16_shapes_off_the_8_element_grid(ops, M, K, N, layout):
    """tensor_linear takes any shape (srcs/ops/mm_ops.hpp:206-232): f16 problems whose K or N is not a multiple of 8 (what TMA
    cannot address) run on the SIMT kernel and must meet the same rule."""
    r = np.random.default_rng(M + K + N)
    x = f16v(r.standard_normal((M, K), np.float32))
    w = f16v(r.standard_normal((K, N), np.float32) * 0.05)
    wd = dev(w if layout == "KN" else np.ascontiguousarray(w.T), torch.float16)
    y = ops.tensor_linear(dev(x, torch.float16), wd, w_layout=ops.W_KN if layout == "KN" else ops.W_NK)
    want = (x.astype(np.float64) @ w.astype(np.float64)).astype(np.float32)
    assert_close_f16(host(y), want, f"linear {M}x{K}x{N} {layout}")


def test_bounded_wait_gives_up_and_the_context_stays_usable(ops):
    """The give-up path of the device-side waits, driven by a condition made on the host: the producer of the single-CTA GEMM
    kernel is told to skip the last K-block of every tile and the waits of that launch poll at most 20000 times. The
    MMA-issuing thread's wait runs out, the kernel records the site and returns (no trap, no fault); the library reports
    B200_ERR_DEVICE_TIMEOUT once, and the next ordinary call on the same context is correct."""
    import ctypes
    from anygpu_b200 import capi
    lib = capi.load()
    r = np.random.default_rng(3)
    M, K, N = 200, 512, 192
    x = f16v(r.standard_normal((M, K), np.float32))
    w = f16v(r.standard_normal((K, N), np.float32) * 0.05)
    xd, wd = dev(x, torch.float16), dev(w, torch.float16)
    yd = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.b200_last_device_error(stream, None) == 0
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.b200_debug_linear_starved_producer(p(xd), K, p(wd), capi.W_KN, p(yd), N, M, K, N, 20000, stream)
    assert rc == 0, rc  # the launch itself succeeds
    detail = ctypes.c_uint32(0)
    assert lib.b200_last_device_error(stream, ctypes.byref(detail)) == -4  # B200_ERR_DEVICE_TIMEOUT
    site = detail.value >> 16
    assert site in (2, 4), hex(detail.value)  # the MMA thread's wait for a full stage (or an epilogue warp that noticed first)
    assert lib.b200_last_device_error(stream, None) == 0  # reading the error word clears it
    torch.cuda.synchronize()
    y = ops.tensor_linear(xd, wd)  # the same kernel, ordinary call
    want = (x.astype(np.float64) @ w.astype(np.float64)).astype(np.float32)
    assert_close_f16(host(y), want, "linear after a timed-out launch")
    assert lib.b200_last_device_error(stream, None) == 0


def test_linear_f16_strided_rows(ops):
    r = np.random.default_rng(9)
    wide = f16v(r.standard_normal((96, 1064), np.float32))
    w = f16v(r.standard_normal((512, 256), np.float32) * 0.05)
    wd = dev(wide, torch.float16)
    y = ops.tensor_linear(wd[:, 16:528], dev(w, torch.float16))
    want = wide[:, 16:528].astype(np.float64) @ w.astype(np.float64)
    assert_close_f16(host(y), want.astype(np.float32), "strided x rows")


# ---- SSD chunked scan ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["ssd_cfg0_shape", "ssd_groups_init", "ssd_ragged_len", "ssd_single_chunk"])
def test_ssd_f32_golden(ops, golden_dir, name):
    g = load(golden_dir, name)
    init = dev(g["initial_states"]) if "initial_states" in g.files else None
    y, fs = ops.tensor_mamba_chunk_scan_combined(dev(g["x"]), dev(g["dt"]), dev(g["A"]), dev(g["B"]), dev(g["C"]), int(g["chunk"]),
                                                 D=dev(g["D"]), dt_bias=dev(g["dt_bias"]), initial_states=init)
    # pass rule of the reference's own SSD checks: abs 1e-3 or rel 1e-2 (scripts/zamba2/mamba_chunk_scan_comb.py:345-347)
    assert_abs(host(y), g["y"], name + " y", 1e-3)
    assert_abs(host(fs), g["final_states"], name + " final_states", 1e-4)


@pytest.fixture(params=["staged", "fused"])
def ssd_path(request):
    """Runs a scan test twice: through the staged kernels (chunk state, state passing, chunk scan) and through the one-kernel
    scan (taken where it covers the shape; the library otherwise chooses by problem size)."""
    old = os.environ.get("B200_SSD_FUSED")
    os.environ["B200_SSD_FUSED"] = "1" if request.param == "fused" else "0"
    yield request.param
    if old is None:
        os.environ.pop("B200_SSD_FUSED", None)
    else:
        os.environ["B200_SSD_FUSED"] = old


def _ssd_inputs(seed, b, l, H, P, G, N):
    r = np.random.default_rng(seed)
    x = r.standard_normal((b, l, H, P), np.float32) * 0.5
    dt = r.standard_normal((b, l, H), np.float32)
    A = -r.uniform(1.0, 16.0, H).astype(np.float32)
    B = r.standard_normal((b, l, G, N), np.float32) * 0.5
    C = r.standard_normal((b, l, G, N), np.float32) * 0.5
    D = np.ones(H, np.float32)
    dtv = np.exp(r.uniform(np.log(1e-3), np.log(1e-1), H))
    dt_bias = (dtv + np.log(-np.expm1(-dtv))).astype(np.float32)
    return x, dt, A, B, C, D, dt_bias


@pytest.mark.parametrize("dims", [(1, 512, 4, 64, 1, 64, 256), (2, 256, 8, 64, 2, 64, 128), (1, 300, 4, 64, 1, 64, 256),
                                  (1, 128, 2, 64, 1, 128, 64), (2, 64, 8, 64, 1, 16, 32), (1, 96, 2, 32, 1, 16, 32),
                                  (1, 256, 2, 64, 1, 128, 128), (1, 512, 4, 64, 2, 128, 256), (3, 1024, 16, 64, 1, 64, 256),
                                  (1, 200, 12, 64, 3, 64, 128), (2, 640, 6, 64, 2, 64, 256), (5, 100, 3, 64, 1, 64, 256)])
def test_ssd_f16_vs_oracle(ops, dims, ssd_path):
    b, l, H, P, G, N, Q = dims
    x, dt, A, B, C, D, dt_bias = _ssd_inputs(sum(dims), b, l, H, P, G, N)
    x, dt, B, C = map(f16v, (x, dt, B, C))
    init = (np.random.default_rng(1).standard_normal((b, H, P, N), np.float32) * 0.1).astype(np.float32)
    h = torch.float16
    y, fs = ops.tensor_mamba_chunk_scan_combined(dev(x, h), dev(dt, h), dev(A), dev(B, h), dev(C, h), Q, D=dev(D), dt_bias=dev(dt_bias),
                                                 initial_states=dev(init))
    wy, wfs = orc.ssd_chunk_scan(x, dt, A, B, C, Q, D=D, dt_bias=dt_bias, initial_states=init)
    assert_close_f16(host(y), wy, f"ssd y {dims}")
    assert_close_f16(host(fs), wfs, f"ssd final_states {dims}")


def test_ssd_f16_in_place_slices(ops, ssd_path):
    # x | B | C read in place from one [b,l,conv_dim] tensor and dt from another wide tensor, as the mixer does
    b, l, H, P, G, N, Q = 2, 384, 4, 64, 1, 64, 128
    x, dt, A, B, C, D, dt_bias = _ssd_inputs(77, b, l, H, P, G, N)
    x, dt, B, C = map(f16v, (x, dt, B, C))
    xbc = np.concatenate([x.reshape(b, l, H * P), B.reshape(b, l, G * N), C.reshape(b, l, G * N)], axis=2)
    wide_dt = np.concatenate([np.zeros((b, l, 24), np.float32), dt], axis=2)
    xd, dd = dev(xbc, torch.float16), dev(wide_dt, torch.float16)
    y, fs = ops.tensor_mamba_chunk_scan_combined(xd[:, :, :H * P].unflatten(2, (H, P)), dd[:, :, 24:], dev(A),
                                                 xd[:, :, H * P:H * P + G * N].unflatten(2, (G, N)),
                                                 xd[:, :, H * P + G * N:].unflatten(2, (G, N)), Q, D=dev(D), dt_bias=dev(dt_bias))
    wy, wfs = orc.ssd_chunk_scan(x, dt, A, B, C, Q, D=D, dt_bias=dt_bias)
    assert_close_f16(host(y), wy, "ssd in-place y")
    assert_close_f16(host(fs), wfs, "ssd in-place final_states")


def test_ssd_fused_matches_staged_and_state_in_place(ops):
    """The one-kernel scan against the staged kernels on the same inputs (both round the same operands to f16, so they agree far
    inside the oracle tolerance), and final_states written over initial_states (the chunked-prefill calling pattern)."""
    b, l, H, P, G, N, Q = 3, 900, 8, 64, 2, 64, 256
    x, dt, A, B, C, D, dt_bias = _ssd_inputs(5, b, l, H, P, G, N)
    h = torch.float16
    init = dev(np.random.default_rng(2).standard_normal((b, H, P, N), np.float32) * 0.1)
    args = (dev(x, h), dev(dt, h), dev(A), dev(B, h), dev(C, h), Q)
    kw = dict(D=dev(D), dt_bias=dev(dt_bias))
    res = {}
    for mode in ("0", "1"):
        os.environ["B200_SSD_FUSED"] = mode
        try:
            res[mode] = ops.tensor_mamba_chunk_scan_combined(*args, initial_states=init, exact_final_state=True, **kw)
        finally:
            os.environ.pop("B200_SSD_FUSED", None)
    assert_close_f16(host(res["1"][0]), host(res["0"][0]), "fused vs staged y")
    assert rel_l2(host(res["1"][0]), host(res["0"][0])) < 1e-3
    assert_abs(host(res["1"][1]), host(res["0"][1]), "fused vs staged final state", 2e-3)
    os.environ["B200_SSD_FUSED"] = "1"
    try:
        st = init.clone()
        ops.tensor_mamba_chunk_scan_combined(*args, initial_states=st, final_states_out=st, exact_final_state=True, **kw)
    finally:
        os.environ.pop("B200_SSD_FUSED", None)
    assert torch.equal(st, res["1"][1])


# ---- decode recurrence --------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dims", [(3, 8, 64, 1, 64), (2, 4, 64, 2, 128), (2, 8, 64, 1, 16), (1, 2, 8, 1, 24), (2, 4, 32, 1, 64),
                                  (2, 4, 40, 2, 64), (2, 3, 16, 1, 32), (1, 2, 128, 1, 16), (2, 2, 8, 1, 64), (1, 2, 100, 1, 32)])
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_selective_state_update_steps(ops, dims, dtype):
    b, H, P, G, N = dims
    steps = 5
    x, dt, A, B, C, D, dt_bias = _ssd_inputs(sum(dims), b, steps, H, P, G, N)
    td = torch.float16 if dtype == "f16" else torch.float32
    if dtype == "f16":
        x, dt, B, C = map(f16v, (x, dt, B, C))
    st0 = (np.random.default_rng(4).standard_normal((b, H, P, N), np.float32) * 0.1).astype(np.float32)
    wy, wst = orc.ssd_recurrence(x, dt, A, B, C, D=D, dt_bias=dt_bias, state=st0)
    st = dev(st0)
    Ad, Dd, bd = dev(A), dev(D), dev(dt_bias)
    ys = [host(ops.tensor_mamba_selective_state_update(st, dev(x[:, t], td), dev(dt[:, t], td), Ad, dev(B[:, t], td), dev(C[:, t], td),
                                                       D=Dd, dt_bias=bd)) for t in range(steps)]
    got = np.stack(ys, axis=1)
    if dtype == "f16":
        assert_close_f16(got, wy, "decode y")
    else:
        assert_abs(got, wy, "decode y", 1e-4)
    assert_abs(host(st), wst, "decode state", 1e-4)


@pytest.mark.parametrize("shape", [(13, 520), (3, 7, 2560), (5, 36), (2, 8200), (4, 8192)])
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_rms_norm(ops, shape, dtype):
    r = np.random.default_rng(21)
    x = (r.standard_normal(shape) * 1.5).astype(np.float32)
    w = (1.0 + 0.2 * r.standard_normal(shape[-1])).astype(np.float32)
    td = torch.float16 if dtype == "f16" else torch.float32
    if dtype == "f16":
        x, w = f16v(x), f16v(w)
    for zc in (False, True):
        got = ops.tensor_rms_norm(torch.from_numpy(x).cuda().to(td), torch.from_numpy(w).cuda().to(td), 1e-5, zero_centered=zc)
        want = orc.rms_norm(x, w, 1e-5, zero_centered=zc)
        if dtype == "f16":
            assert_close_f16(got.float().cpu().numpy(), want, f"rms_norm f16 zero_centered={zc}")
        else:
            assert_abs(got.cpu().numpy(), want, f"rms_norm f32 zero_centered={zc}", 1e-4)


def test_rms_norm_golden_from_reference(ops, golden_dir):
    g = np.load(os.path.join(golden_dir, "rms_norm.npz"))
    got = ops.tensor_rms_norm(torch.from_numpy(g["x"]).cuda(), torch.from_numpy(g["w"]).cuda(), float(g["eps"]))
    assert_abs(got.cpu().numpy(), g["y_ref"], "rms_norm vs the reference CPU operator", 1e-4)


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_ssd_ragged_length_final_state_modes(ops, dtype, ssd_path):
    """seqlen % chunk != 0: y is exact in both modes; final_states follows the reference script (padded tail decays it) by
    default and is the state after the last real token with exact_final_state."""
    b, l, H, P, G, N, Q = 2, 300, 4, 64, 1, 64, 128
    r = np.random.default_rng(31)
    x = (r.standard_normal((b, l, H, P)) * 0.5).astype(np.float32)
    dt = r.standard_normal((b, l, H)).astype(np.float32)
    Bm = (r.standard_normal((b, l, G, N)) * 0.5).astype(np.float32)
    Cm = (r.standard_normal((b, l, G, N)) * 0.5).astype(np.float32)
    A = -(r.uniform(1, 16, H)).astype(np.float32)
    D, dtb = np.ones(H, np.float32), np.full(H, -2.0, np.float32)
    td = torch.float16 if dtype == "f16" else torch.float32
    if dtype == "f16":
        x, dt, Bm, Cm = f16v(x), f16v(dt), f16v(Bm), f16v(Cm)
    dev = lambda a, t=td: torch.from_numpy(a).cuda().to(t)
    args = (dev(x), dev(dt), dev(A, torch.float32), dev(Bm), dev(Cm), Q)
    kw = dict(D=dev(D, torch.float32), dt_bias=dev(dtb, torch.float32))
    y1, fs_ref_mode = ops.tensor_mamba_chunk_scan_combined(*args, **kw)
    y2, fs_exact = ops.tensor_mamba_chunk_scan_combined(*args, exact_final_state=True, **kw)
    assert torch.equal(y1, y2)
    wy, wfs_script = orc.ssd_chunk_scan(x, dt, A, Bm, Cm, Q, D=D, dt_bias=dtb)         # restates the script, padding included
    _, wfs_true = orc.ssd_recurrence(x, dt, A, Bm, Cm, D=D, dt_bias=dtb)                # token-by-token recurrence
    assert np.abs(wfs_script - wfs_true).max() > 1e-3                                   # the two really differ on this input
    if dtype == "f16":
        assert_close_f16(y1.float().cpu().numpy(), wy, "ragged y")
        assert_close_f16(fs_ref_mode.cpu().numpy(), wfs_script, "final state, script mode")
        assert_close_f16(fs_exact.cpu().numpy(), wfs_true, "final state, exact mode")
    else:
        assert_abs(y1.cpu().numpy(), wy, "ragged y", 1e-3)
        assert_abs(fs_ref_mode.cpu().numpy(), wfs_script, "final state, script mode", 1e-4)
        assert_abs(fs_exact.cpu().numpy(), wfs_true, "final state, exact mode", 1e-4)
