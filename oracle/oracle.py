"""numpy front-end of the CPU oracle (``liboracle.so``) and, when it was built, of the reference's
own CPU operators (``_ref/libanygpu_ref.so``).

TEST INFRASTRUCTURE ONLY. Imported by ``tests/``, by the smoke check and by the benchmark's CPU-baseline
leg. The shipped package never imports this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

_f32p = ctypes.POINTER(ctypes.c_float)
_i64 = ctypes.c_int64


def reference_checkout():
    """Where the anyGPU checkout lies: the environment variable ANYGPU_REF, else a directory named `reference` beside this
    repository. None when neither holds the sources."""
    root = os.path.dirname(_HERE)
    for cand in (os.environ.get("ANYGPU_REF"), os.path.join(os.path.dirname(root), "reference")):
        if cand and os.path.exists(os.path.join(cand, "srcs", "core", "core.cpp")):
            return os.path.abspath(cand)
    return None


def build(with_ref=True):
    """Compile liboracle.so (always) and, only where the anyGPU checkout exists, _ref/libanygpu_ref.so (its CPU operators) and
    _ref/ref_cuda_bench (a timing program around its CUDA kernels)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "all"])
    ref = reference_checkout()
    if with_ref and ref is not None:
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF={ref}"])
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref_cuda", f"REF={ref}"])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build(with_ref=False)
        _LIB = ctypes.CDLL(path)
        _LIB.orc_num_threads.restype = ctypes.c_int
    return _LIB


def ref_lib():
    """The reference's own CPU operators, or None when they were not built."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libanygpu_ref.so")
        if not os.path.exists(path):
            return None
        _REF = ctypes.CDLL(path)
    return _REF


def _p(a):
    if a is None:
        return ctypes.cast(None, _f32p)
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(_f32p)


def _c(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def set_num_threads(n):
    lib().orc_set_num_threads(ctypes.c_int(n))


def num_threads():
    return lib().orc_num_threads()


def round_f16(a):
    """Round an fp32 array through binary16 (what writing an f16 tensor does)."""
    return np.asarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)


def linear(x, w, fast=True):
    x, w = _c(x), _c(w)
    K, N = w.shape
    M = x.size // K
    y = np.empty(x.shape[:-1] + (N,), np.float32)
    fn = lib().orc_linear_f32_fast if fast else lib().orc_linear_f32
    fn(_p(x), _p(w), _p(y), _i64(M), _i64(K), _i64(N))
    return y


def causal_conv1d(x, w, b):
    """x (batch, dims, seq_len), w (dims, width), b (dims)."""
    x, w, b = _c(x), _c(w), _c(b)
    B, D, S = x.shape
    y = np.empty_like(x)
    lib().orc_causal_conv1d_f32(_p(x), _p(w), _p(b), _p(y), _i64(B), _i64(D), _i64(S), _i64(w.shape[1]))
    return y


def causal_conv1d_update(x_t, conv_state, w, b):
    """x_t (batch, dims); conv_state (batch, dims, width-1) fp32, advanced IN PLACE. Returns y_t."""
    x_t, w, b = _c(x_t), _c(w), _c(b)
    assert conv_state.dtype == np.float32 and conv_state.flags["C_CONTIGUOUS"]
    B, D = x_t.shape
    y = np.empty_like(x_t)
    lib().orc_causal_conv1d_update_f32(_p(x_t), _p(conv_state), _p(w), _p(b), _p(y), _i64(B), _i64(D), _i64(w.shape[1]))
    return y


def gated_rmsnorm(x, z, w, eps, gsize=None):
    x, z, w = _c(x), _c(z), _c(w)
    d = x.shape[-1]
    rows = x.size // d
    y = np.empty_like(x)
    lib().orc_gated_rmsnorm_f32(_p(x), _p(z), _p(w), _p(y), _i64(rows), _i64(d), _i64(gsize or d), ctypes.c_float(eps))
    return y


def rms_norm(x, w, eps, zero_centered=False):
    x, w = _c(x), _c(w)
    d = x.shape[-1]
    y = np.empty_like(x)
    lib().orc_rms_norm_f32(_p(x), _p(w), _p(y), _i64(x.size // d), _i64(d), ctypes.c_float(eps), ctypes.c_int(int(zero_centered)))
    return y


def _r16(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


def decoder_prefill(hidden, wts, input_norm_weight, rms_eps, cfg, f16io=False):
    """The Mamba decoder layer around the mixer: hidden + mixer(rms_norm(hidden) * w_in). With f16io every operator's output
    tensor is rounded to binary16 (norm output, mixer stages, and the sum)."""
    normed = rms_norm(hidden, input_norm_weight, rms_eps)
    if f16io:
        normed = _r16(normed)
    res = mixer_prefill(normed, wts, cfg, f16io=f16io)
    out = np.asarray(hidden, np.float32) + res["out"]
    res["out"] = _r16(out) if f16io else out
    return res


def decoder_decode(hidden_t, wts, input_norm_weight, rms_eps, cfg, conv_state, ssm_state, f16io=False):
    normed = rms_norm(hidden_t, input_norm_weight, rms_eps)
    if f16io:
        normed = _r16(normed)
    out = np.asarray(hidden_t, np.float32) + mixer_decode(normed, wts, cfg, conv_state, ssm_state, f16io=f16io)
    return _r16(out) if f16io else out


def ssd_chunk_scan(x, dt, A, B, C, chunk, D=None, dt_bias=None, initial_states=None, dt_softplus=True):
    """Argument order of mamba_chunk_scan_combined_ref. Returns (y [b,l,H,P], final_states [b,H,P,N])."""
    x, dt, A, B, C, D, dt_bias, initial_states = map(_c, (x, dt, A, B, C, D, dt_bias, initial_states))
    b, l, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    y = np.empty_like(x)
    fs = np.empty((b, H, P, N), np.float32)
    lib().orc_ssd_chunk_scan_f32(_p(x), _p(dt), _p(A), _p(B), _p(C), _p(D), _p(dt_bias), _p(initial_states), _p(y), _p(fs),
                                 _i64(b), _i64(l), _i64(H), _i64(P), _i64(G), _i64(N), _i64(chunk), ctypes.c_int(int(dt_softplus)))
    return y, fs


def ssd_recurrence(x, dt, A, B, C, D=None, dt_bias=None, state=None, dt_softplus=True):
    """Token-by-token recurrence. state [b,H,P,N] (copied; zeros when None). Returns (y, final_state)."""
    x, dt, A, B, C, D, dt_bias = map(_c, (x, dt, A, B, C, D, dt_bias))
    b, l, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    st = np.zeros((b, H, P, N), np.float32) if state is None else np.array(state, dtype=np.float32, order="C")
    y = np.empty_like(x)
    lib().orc_ssd_recurrence_f32(_p(x), _p(dt), _p(A), _p(B), _p(C), _p(D), _p(dt_bias), _p(st), _p(y),
                                 _i64(b), _i64(l), _i64(H), _i64(P), _i64(G), _i64(N), ctypes.c_int(int(dt_softplus)))
    return y, st


def mixer_prefill(u, wts, cfg, initial_states=None, f16io=False, want_intermediates=False):
    """u [b,l,d_model]; wts dict with in_proj_weight [d_model,d_in_proj], conv1d_weight [conv_dim,W], conv1d_bias,
    dt_bias, A_log, D, norm_weight, out_proj_weight [d_inner,d_model]; cfg dict with d_inner, nheads, headdim, ngroups,
    d_state, d_conv, chunk, eps and optional norm_group_size.
    Returns dict(out, final_state, conv_state[, zxbcdt, xbc, y, g])."""
    u = _c(u)
    b, l, d_model = u.shape
    d_inner, H, P, G, N = cfg["d_inner"], cfg["nheads"], cfg["headdim"], cfg["ngroups"], cfg["d_state"]
    W, Q = cfg["d_conv"], cfg["chunk"]
    conv_dim = d_inner + 2 * G * N
    d_in_proj = 2 * d_inner + 2 * G * N + H
    T = b * l
    res = {"out": np.empty((b, l, d_model), np.float32), "final_state": np.empty((b, H, P, N), np.float32),
           "conv_state": np.empty((b, conv_dim, W - 1), np.float32)}
    if want_intermediates:
        res.update(zxbcdt=np.empty((b, l, d_in_proj), np.float32), xbc=np.empty((b, l, conv_dim), np.float32),
                   y=np.empty((b, l, d_inner), np.float32), g=np.empty((b, l, d_inner), np.float32))
    w = {k: _c(v) for k, v in wts.items()}
    init = _c(initial_states)
    lib().orc_mamba2_mixer_prefill_f32(
        _p(u), _p(w["in_proj_weight"]), _p(w["conv1d_weight"]), _p(w["conv1d_bias"]), _p(w["dt_bias"]), _p(w["A_log"]),
        _p(w["D"]), _p(w["norm_weight"]), _p(w["out_proj_weight"]), _p(init),
        _p(res["out"]), _p(res.get("zxbcdt")), _p(res.get("xbc")), _p(res.get("y")), _p(res.get("g")),
        _p(res["final_state"]), _p(res["conv_state"]),
        _i64(b), _i64(l), _i64(d_model), _i64(d_inner), _i64(H), _i64(P), _i64(G), _i64(N), _i64(W), _i64(Q),
        _i64(cfg.get("norm_group_size") or d_inner), ctypes.c_float(cfg["eps"]), ctypes.c_int(int(f16io)))
    assert T == b * l
    return res


def mixer_decode(u_t, wts, cfg, conv_state, ssm_state, f16io=False):
    """u_t [b,d_model]; conv_state [b,conv_dim,W-1] and ssm_state [b,H,P,N] fp32, advanced IN PLACE. Returns out [b,d_model]."""
    u_t = _c(u_t)
    b, d_model = u_t.shape
    d_inner, H, P, G, N = cfg["d_inner"], cfg["nheads"], cfg["headdim"], cfg["ngroups"], cfg["d_state"]
    W = cfg["d_conv"]
    for s in (conv_state, ssm_state):
        assert s.dtype == np.float32 and s.flags["C_CONTIGUOUS"]
    w = {k: _c(v) for k, v in wts.items()}
    out = np.empty((b, d_model), np.float32)
    lib().orc_mamba2_mixer_decode_f32(
        _p(u_t), _p(w["in_proj_weight"]), _p(w["conv1d_weight"]), _p(w["conv1d_bias"]), _p(w["dt_bias"]), _p(w["A_log"]),
        _p(w["D"]), _p(w["norm_weight"]), _p(w["out_proj_weight"]), _p(conv_state), _p(ssm_state), _p(out),
        _i64(b), _i64(d_model), _i64(d_inner), _i64(H), _i64(P), _i64(G), _i64(N), _i64(W),
        _i64(cfg.get("norm_group_size") or d_inner), ctypes.c_float(cfg["eps"]), ctypes.c_int(int(f16io)))
    return out


# ---- the reference's own CPU operators (None when not built) -------------------------------------------------

def ref_linear(x, w):
    r = ref_lib()
    x, w = _c(x), _c(w)
    K, N = w.shape
    M = x.size // K
    y = np.empty(x.shape[:-1] + (N,), np.float32)
    r.ref_linear_f32(_p(x), _p(w), _p(y), ctypes.c_longlong(M), ctypes.c_longlong(K), ctypes.c_longlong(N))
    return y


def ref_causal_conv1d(x, w, b):
    r = ref_lib()
    x, w, b = _c(x), _c(w), _c(b)
    B, D, S = x.shape
    y = np.empty_like(x)
    r.ref_causal_conv1d_f32(_p(x), _p(w), _p(b), _p(y), ctypes.c_longlong(B), ctypes.c_longlong(D), ctypes.c_longlong(S),
                            ctypes.c_longlong(w.shape[1]))
    return y


def ref_gated_rmsnorm(x, z, w, eps, gsize=0):
    r = ref_lib()
    x, z, w = _c(x), _c(z), _c(w)
    d = x.shape[-1]
    y = np.empty_like(x)
    r.ref_gated_rmsnorm_f32(_p(x), _p(z), _p(w), _p(y), ctypes.c_longlong(x.size // d), ctypes.c_longlong(d),
                            ctypes.c_int(gsize or d), ctypes.c_float(eps))
    return y


def ref_rms_norm(x, w, eps):
    r = ref_lib()
    x, w = _c(x), _c(w)
    d = x.shape[-1]
    y = np.empty_like(x)
    r.ref_rms_norm_f32(_p(x), _p(w), _p(y), ctypes.c_longlong(x.size // d), ctypes.c_longlong(d), ctypes.c_float(eps))
    return y
