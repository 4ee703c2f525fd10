"""Generates the golden vectors under tests/golden/ from the anyGPU reference itself.

Run once in a container that has the anyGPU checkout (its location: $ANYGPU_REF, see REF below):

    python tests/golden/make_golden.py

Sources of truth, all executed unmodified from the checkout:
  * scripts/zamba2/mamba_chunk_scan_comb.py : mamba_chunk_scan_combined_ref (torch, CPU)        -> ssd_*.npz
  * the formula of scripts/fused_test_cases.py:41 (silu(conv1d(...))[..., :seq_len]) in torch
    and tensor_causal_conv1d<float32,CPU> compiled from srcs/fused/causal_conv1d.hpp             -> conv1d_*.npz
  * tensor_zamba_gated_rmsnorm<float32,CPU>, tensor_linear<float32,CPU> compiled from the srcs   -> gated_rmsnorm.npz, linear.npz
  * the composition of those pieces into one Mamba2 mixer layer at the configuration-0 sizes     -> mixer_cfg0.npz

The compiled pieces come from oracle/_ref/libanygpu_ref.so (built by `make -C oracle ref`).
The committed .npz files are what the tests read; the checkout is not needed to run the tests.
"""
import contextlib
import io
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as _orc_for_ref  # noqa: E402

REF = _orc_for_ref.reference_checkout()
if REF is None:
    raise SystemExit("the anyGPU checkout is needed to regenerate the golden vectors: set ANYGPU_REF to its path")
sys.path.insert(0, os.path.join(REF, "scripts", "dnn_inspector"))
sys.path.insert(0, os.path.join(REF, "scripts", "zamba2"))

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

import mamba_chunk_scan_comb as refpy  # noqa: E402  (the reference's script)
from oracle import oracle as orc  # noqa: E402
from anygpu_b200 import synth  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def ref_ssd(x, dt, A, B, C, chunk, D, dt_bias, init):
    t = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a))
    with contextlib.redirect_stdout(io.StringIO()):  # the script prints shapes
        y, fs = refpy.mamba_chunk_scan_combined_ref(t(x), t(dt), t(A), t(B), t(C), chunk, D=t(D), dt_bias=t(dt_bias),
                                                    initial_states=t(init), dt_softplus=True)
    return y.numpy(), fs.numpy()


def ssd_case(name, seed, b, l, H, P, G, N, chunk, with_init):
    r = np.random.default_rng(seed)
    x = r.standard_normal((b, l, H, P), np.float32)
    dt = r.standard_normal((b, l, H), np.float32)
    A = -r.uniform(1.0, 16.0, H).astype(np.float32)
    B = r.standard_normal((b, l, G, N), np.float32)
    C = r.standard_normal((b, l, G, N), np.float32)
    D = r.standard_normal(H).astype(np.float32)
    dtv = np.exp(r.uniform(np.log(1e-3), np.log(1e-1), H))
    dt_bias = (dtv + np.log(-np.expm1(-dtv))).astype(np.float32)
    init = (r.standard_normal((b, H, P, N), np.float32) * np.float32(0.1)) if with_init else None
    y, fs = ref_ssd(x, dt, A, B, C, chunk, D, dt_bias, init)
    d = dict(x=x, dt=dt, A=A, B=B, C=C, D=D, dt_bias=dt_bias, chunk=np.int64(chunk), y=y, final_states=fs)
    if with_init:
        d["initial_states"] = init
    np.savez(os.path.join(OUT, name + ".npz"), **d)
    print(name, "y", y.shape, "max|y|", np.abs(y).max())


def conv_case(name, seed, b, d, s, w):
    r = np.random.default_rng(seed)
    x = r.standard_normal((b, d, s), np.float32)
    wt = r.standard_normal((d, w), np.float32)
    bs = r.standard_normal((d,), np.float32)
    tx, tw, tb = map(torch.from_numpy, (x, wt, bs))
    y_torch = F.silu(F.conv1d(tx, tw.unsqueeze(1), tb, stride=1, padding=w - 1, groups=d))[:, :, :s].numpy()
    y_ref = orc.ref_causal_conv1d(x, wt, bs)
    np.savez(os.path.join(OUT, name + ".npz"), x=x, w=wt, b=bs, y_torch=y_torch, y_ref=y_ref)
    print(name, "max|torch-ref|", np.abs(y_torch - y_ref).max())


def norm_case(name, seed, rows, d, eps):
    r = np.random.default_rng(seed)
    x = r.standard_normal((rows, d), np.float32)
    z = r.standard_normal((rows, d), np.float32)
    w = r.standard_normal((d,), np.float32)
    y_ref = orc.ref_gated_rmsnorm(x, z, w, eps, gsize=d)
    g = torch.from_numpy(x) * F.silu(torch.from_numpy(z))
    y_torch = (g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + eps) * torch.from_numpy(w)).numpy()
    np.savez(os.path.join(OUT, name + ".npz"), x=x, z=z, w=w, eps=np.float32(eps), y_ref=y_ref, y_torch=y_torch)
    print(name, "max|torch-ref|", np.abs(y_torch - y_ref).max())


def linear_case(name, seed, M, K, N):
    r = np.random.default_rng(seed)
    x = r.standard_normal((M, K), np.float32)
    w = r.standard_normal((K, N), np.float32)
    y_ref = orc.ref_linear(x, w)
    np.savez(os.path.join(OUT, name + ".npz"), x=x, w=w, y_ref=y_ref)
    print(name, "max|np-ref|", np.abs(x @ w - y_ref).max())


def rms_norm_case(name, seed, rows, d, eps):
    r = np.random.default_rng(seed)
    x = r.standard_normal((rows, d), np.float32) * 1.5
    w = r.standard_normal((d,), np.float32)
    y_ref = orc.ref_rms_norm(x, w, eps)
    xt = torch.from_numpy(x)
    y_torch = (xt * torch.rsqrt(xt.pow(2).mean(-1, keepdim=True) + eps) * torch.from_numpy(w)).numpy()
    np.savez(os.path.join(OUT, name + ".npz"), x=x, w=w, eps=np.float32(eps), y_ref=y_ref, y_torch=y_torch)
    print(name, "max|torch-ref|", np.abs(y_torch - y_ref).max())


def decoder_cfg0():
    """The decoder layer around the cfg0 mixer, every stage run by reference code: hidden + mixer(rms_norm(hidden) * w_in)."""
    cfg = synth.CONFIGS["cfg0"]
    w = synth.make_weights(cfg, seed=0)
    hidden = synth.make_input(cfg, seed=0)
    w_in = (1.0 + 0.1 * np.random.default_rng(99).standard_normal(cfg["d_model"])).astype(np.float32)
    normed = orc.ref_rms_norm(hidden, w_in, 1e-5)
    m = ref_mixer(normed, w, cfg)
    np.savez(os.path.join(OUT, "decoder_cfg0.npz"), input_norm_weight=w_in, rms_eps=np.float32(1e-5), normed=normed,
             out=hidden + m["out"], final_states=m["final_states"])
    print("decoder_cfg0 max|out|", np.abs(hidden + m["out"]).max())


def mixer_cfg0():
    """One Mamba2 mixer layer at the configuration-0 sizes, every stage run by reference code."""
    cfg = synth.CONFIGS["cfg0"]
    w = synth.make_weights(cfg, seed=0)
    u = synth.make_input(cfg, seed=0)
    m = ref_mixer(u, w, cfg)
    # inputs are regenerated from the seed by the tests; keep checksums so a generator drift is caught
    chk = np.array([np.float64(np.abs(v).sum()) for v in [u] + [w[k] for k in sorted(w)]])
    np.savez(os.path.join(OUT, "mixer_cfg0.npz"), input_checksums=chk, **m)
    print("mixer_cfg0 out", m["out"].shape, "max|out|", np.abs(m["out"]).max(), "max|y|", np.abs(m["y"]).max())


def ref_mixer(u, w, cfg):
    """The mixer composed of the reference's own functions (compiled CPU operators + its Python SSD)."""
    b, l = u.shape[0], u.shape[1]
    d_inner, H, P, G, N = cfg["d_inner"], cfg["nheads"], cfg["headdim"], cfg["ngroups"], cfg["d_state"]
    conv_dim, d_in_proj = synth.dims(cfg)
    zx = orc.ref_linear(u.reshape(b * l, -1), w["in_proj_weight"]).reshape(b, l, d_in_proj)
    z = zx[..., :d_inner]
    xbc = zx[..., d_inner:d_inner + conv_dim]
    dt = zx[..., d_inner + conv_dim:]
    xbc_c = orc.ref_causal_conv1d(np.ascontiguousarray(xbc.transpose(0, 2, 1)), w["conv1d_weight"], w["conv1d_bias"])
    xbc_c = np.ascontiguousarray(xbc_c.transpose(0, 2, 1))
    x = xbc_c[..., :d_inner].reshape(b, l, H, P)
    Bm = xbc_c[..., d_inner:d_inner + G * N].reshape(b, l, G, N)
    Cm = xbc_c[..., d_inner + G * N:].reshape(b, l, G, N)
    A = -np.exp(w["A_log"])
    y, fs = ref_ssd(x, np.ascontiguousarray(dt), A, Bm, Cm, cfg["chunk"], w["D"], w["dt_bias"], None)
    g = orc.ref_gated_rmsnorm(y.reshape(b * l, d_inner), np.ascontiguousarray(z).reshape(b * l, d_inner), w["norm_weight"],
                              cfg["eps"], gsize=d_inner)
    out = orc.ref_linear(g, w["out_proj_weight"]).reshape(b, l, -1)
    return dict(out=out, y=y.reshape(b, l, d_inner), final_states=fs, g=g.reshape(b, l, d_inner), zxbcdt=zx)


if __name__ == "__main__":
    assert orc.ref_lib() is not None, "build oracle/_ref first: make -C oracle ref"
    ssd_case("ssd_cfg0_shape", 1, 1, 64, 8, 64, 1, 16, 32, False)
    ssd_case("ssd_groups_init", 2, 2, 96, 4, 16, 2, 8, 32, True)
    ssd_case("ssd_ragged_len", 3, 1, 50, 4, 32, 1, 16, 32, False)
    ssd_case("ssd_single_chunk", 4, 1, 16, 2, 8, 1, 8, 16, True)
    conv_case("conv1d_w4", 5, 2, 37, 53, 4)
    conv_case("conv1d_w3", 6, 1, 9, 20, 3)
    conv_case("conv1d_short", 7, 3, 5, 2, 4)
    norm_case("gated_rmsnorm", 8, 6, 512, 1e-5)
    linear_case("linear", 9, 5, 33, 21)
    mixer_cfg0()
    rms_norm_case("rms_norm", 9, 13, 520, 1e-5)
    decoder_cfg0()
