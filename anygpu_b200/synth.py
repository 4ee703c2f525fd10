"""Seeded synthetic weights and inputs for the Mamba2-mixer configurations.

No dataset is involved anywhere on this path: the benchmark configurations are defined by their shapes
and value distributions, and this module is their single definition for the tests and the benchmark.
Tensor ``i`` of a configuration is drawn from ``numpy.random.default_rng(seed + i)`` in the fixed order
``u, in_proj_weight, conv1d_weight, conv1d_bias, dt_bias, A_log, D, norm_weight, out_proj_weight, conv_state,
ssm_state`` so that any subset can be regenerated independently.
"""
import numpy as np

# name -> mixer dimensions. `batch`/`seqlen` are the sizes the configuration is quoted on.
CONFIGS = {
    # single layer, fp32, small enough for the reference CPU path
    "cfg0": dict(batch=1, seqlen=64, d_model=256, d_inner=512, nheads=8, headdim=64, d_state=16, ngroups=1,
                 d_conv=4, chunk=32, eps=1e-5, conv_bias_std=0.0),
    # Zamba2-1.2B-shaped prefill
    "cfg2": dict(batch=4, seqlen=2048, d_model=2048, d_inner=4096, nheads=64, headdim=64, d_state=64, ngroups=1,
                 d_conv=4, chunk=256, eps=1e-5, conv_bias_std=0.0),
    # Zamba2-2.7B-shaped decode
    "cfg3": dict(batch=64, seqlen=1, d_model=2560, d_inner=5120, nheads=80, headdim=64, d_state=64, ngroups=1,
                 d_conv=4, chunk=256, eps=1e-5, conv_bias_std=0.0),
    # Zamba2-7B-shaped prefill
    "cfg4": dict(batch=32, seqlen=4096, d_model=3584, d_inner=7168, nheads=112, headdim=64, d_state=64, ngroups=2,
                 d_conv=4, chunk=256, eps=1e-5, conv_bias_std=0.0),
}

_ORDER = ["u", "in_proj_weight", "conv1d_weight", "conv1d_bias", "dt_bias", "A_log", "D", "norm_weight",
          "out_proj_weight", "conv_state", "ssm_state"]


def dims(cfg):
    conv_dim = cfg["d_inner"] + 2 * cfg["ngroups"] * cfg["d_state"]
    d_in_proj = 2 * cfg["d_inner"] + 2 * cfg["ngroups"] * cfg["d_state"] + cfg["nheads"]
    return conv_dim, d_in_proj


def _rng(seed, name):
    return np.random.default_rng(seed + _ORDER.index(name))


def make_weights(cfg, seed=0):
    """fp32 weights: in/out_proj ~N(0,0.02), conv weight ~N(0,0.5), conv bias 0 (or N(0,std)),
    A_log = log U[1,16], dt_bias = softplus^-1(exp U[log 1e-3, log 1e-1]), D = 1, norm weight 1.
    Projection weights are (in_features, out_features), the layout tensor_linear consumes."""
    conv_dim, d_in_proj = dims(cfg)
    H = cfg["nheads"]
    w = {}
    w["in_proj_weight"] = (_rng(seed, "in_proj_weight").standard_normal((cfg["d_model"], d_in_proj), np.float32) * 0.02)
    w["conv1d_weight"] = (_rng(seed, "conv1d_weight").standard_normal((conv_dim, cfg["d_conv"]), np.float32) * 0.5)
    std = cfg.get("conv_bias_std", 0.0)
    w["conv1d_bias"] = (_rng(seed, "conv1d_bias").standard_normal((conv_dim,), np.float32) * std).astype(np.float32)
    dt = np.exp(_rng(seed, "dt_bias").uniform(np.log(1e-3), np.log(1e-1), H))
    w["dt_bias"] = (dt + np.log(-np.expm1(-dt))).astype(np.float32)
    w["A_log"] = np.log(_rng(seed, "A_log").uniform(1.0, 16.0, H)).astype(np.float32)
    w["D"] = np.ones(H, np.float32)
    w["norm_weight"] = np.ones(cfg["d_inner"], np.float32)
    w["out_proj_weight"] = (_rng(seed, "out_proj_weight").standard_normal((cfg["d_inner"], cfg["d_model"]), np.float32) * 0.02)
    return w


def make_input(cfg, seed=0, batch=None, seqlen=None):
    b = batch or cfg["batch"]
    l = seqlen or cfg["seqlen"]
    return _rng(seed, "u").standard_normal((b, l, cfg["d_model"]), np.float32)


def make_decode_state(cfg, seed=0, batch=None):
    """conv_state [b,conv_dim,d_conv-1] ~N(0,1), ssm_state [b,H,P,N] ~N(0,0.1), both fp32."""
    b = batch or cfg["batch"]
    conv_dim, _ = dims(cfg)
    cs = _rng(seed, "conv_state").standard_normal((b, conv_dim, cfg["d_conv"] - 1), np.float32)
    ss = _rng(seed, "ssm_state").standard_normal((b, cfg["nheads"], cfg["headdim"], cfg["d_state"]), np.float32) * np.float32(0.1)
    return cs, ss


def to_f16_values(a):
    """fp32 array holding exactly the values an f16 copy would hold."""
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


def tp_local_config(cfg, tp):
    """Local mixer sizes of one rank of a head-sharded layer: nheads/tp heads, their share of d_inner and the group(s) they use."""
    H, G = cfg["nheads"], cfg["ngroups"]
    assert H % tp == 0 and cfg["d_inner"] % tp == 0
    Hl, hpg = H // tp, H // G
    assert (Hl <= hpg and hpg % Hl == 0) or (Hl % hpg == 0), "a rank's heads must sit inside one group or cover whole groups"
    Gl = 1 if Hl <= hpg else Hl // hpg
    return dict(cfg, d_inner=cfg["d_inner"] // tp, nheads=Hl, ngroups=Gl, norm_group_size=0)


def shard_weights_tp(w, cfg, tp, rank):
    """Slices of the (in,out)-layout weights that rank `rank` of `tp` owns: in_proj columns z_r | x_r | B,C of its group(s) |
    dt_r (zero-padded to a multiple of 8 columns), conv rows for the same channels, head slices of dt_bias / A_log / D,
    its slice of the norm weight and its rows of out_proj."""
    d_inner, H, G, N = cfg["d_inner"], cfg["nheads"], cfg["ngroups"], cfg["d_state"]
    loc = tp_local_config(cfg, tp)
    dl, Hl, Gl = loc["d_inner"], loc["nheads"], loc["ngroups"]
    hpg = H // G
    g0 = (rank * Hl) // hpg
    ch = np.arange(rank * dl, (rank + 1) * dl)                       # the rank's x / z channels
    grp = np.arange(g0 * N, (g0 + Gl) * N)                           # its B (and C) columns inside the G*N block
    heads = np.arange(rank * Hl, (rank + 1) * Hl)
    conv_rows = np.concatenate([ch, d_inner + grp, d_inner + G * N + grp])
    cols = np.concatenate([ch, d_inner + conv_rows, 2 * d_inner + 2 * G * N + heads])
    w_in = w["in_proj_weight"][:, cols]
    pad = (-w_in.shape[1]) % 8
    if pad:
        w_in = np.concatenate([w_in, np.zeros((w_in.shape[0], pad), w_in.dtype)], axis=1)
    return {
        "in_proj_weight": np.ascontiguousarray(w_in),
        "conv1d_weight": np.ascontiguousarray(w["conv1d_weight"][conv_rows]),
        "conv1d_bias": np.ascontiguousarray(w["conv1d_bias"][conv_rows]),
        "dt_bias": np.ascontiguousarray(w["dt_bias"][heads]),
        "A_log": np.ascontiguousarray(w["A_log"][heads]),
        "D": np.ascontiguousarray(w["D"][heads]),
        "norm_weight": np.ascontiguousarray(w["norm_weight"][ch]),
        "out_proj_weight": np.ascontiguousarray(w["out_proj_weight"][ch]),
    }
