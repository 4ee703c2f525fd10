"""Pins the CPU oracle: against golden vectors generated from the anyGPU reference (its Python SSD script and its
compiled CPU operators), against the reference operators themselves when they were built here, and against an
independent per-token recurrence."""
import os

import numpy as np
import pytest

from anygpu_b200 import synth
from oracle import oracle as orc
from tolerance import assert_abs


def load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name + ".npz"))


@pytest.mark.parametrize("name", ["conv1d_w4", "conv1d_w3", "conv1d_short"])
def test_conv1d_matches_reference_cpu_bit_exact(golden_dir, name):
    g = load(golden_dir, name)
    y = orc.causal_conv1d(g["x"], g["w"], g["b"])
    # same loop order and accumulation type as the reference's CPU operator -> identical bits
    assert np.array_equal(y, g["y_ref"])
    # the reference's own test compares with the torch golden at abs 1e-3 (tests/ext_torch_tests.cpp:745-778)
    assert_abs(y, g["y_torch"], name)


def test_gated_rmsnorm_matches_reference_cpu_bit_exact(golden_dir):
    g = load(golden_dir, "gated_rmsnorm")
    y = orc.gated_rmsnorm(g["x"], g["z"], g["w"], float(g["eps"]))
    assert np.array_equal(y, g["y_ref"])
    assert_abs(y, g["y_torch"], "gated_rmsnorm")


def test_gated_rmsnorm_groups():
    r = np.random.default_rng(0)
    x, z = r.standard_normal((3, 64), np.float32), r.standard_normal((3, 64), np.float32)
    w = r.standard_normal(64).astype(np.float32)
    y = orc.gated_rmsnorm(x, z, w, 1e-5, gsize=16)
    g = x * (z / (1 + np.exp(-z)))
    e = g.reshape(3, 4, 16)
    e = (e / np.sqrt((e ** 2).mean(-1, keepdims=True) + 1e-5)).reshape(3, 64) * w
    assert_abs(y, e, "grouped", 1e-5)


def test_linear_matches_reference_cpu_bit_exact(golden_dir):
    g = load(golden_dir, "linear")
    assert np.array_equal(orc.linear(g["x"], g["w"], fast=False), g["y_ref"])
    assert np.array_equal(orc.linear(g["x"], g["w"], fast=True), g["y_ref"])


@pytest.mark.parametrize("name", ["ssd_cfg0_shape", "ssd_groups_init", "ssd_ragged_len", "ssd_single_chunk"])
def test_ssd_matches_reference_python(golden_dir, name):
    g = load(golden_dir, name)
    init = g["initial_states"] if "initial_states" in g.files else None
    y, fs = orc.ssd_chunk_scan(g["x"], g["dt"], g["A"], g["B"], g["C"], int(g["chunk"]), D=g["D"], dt_bias=g["dt_bias"],
                               initial_states=init)
    # pass rule of the reference's own SSD checks (scripts/zamba2/mamba_chunk_scan_comb.py:345-347) is abs 1e-3 / rel 1e-2;
    # two fp32 evaluations of the same formula agree far better than that
    assert_abs(y, g["y"], name + " y", 2e-4)
    assert_abs(fs, g["final_states"], name + " final_states", 2e-5)


@pytest.mark.parametrize("name", ["ssd_cfg0_shape", "ssd_groups_init", "ssd_single_chunk"])
def test_ssd_chunked_equals_recurrence(golden_dir, name):
    g = load(golden_dir, name)
    init = g["initial_states"] if "initial_states" in g.files else None
    y, fs = orc.ssd_recurrence(g["x"], g["dt"], g["A"], g["B"], g["C"], D=g["D"], dt_bias=g["dt_bias"], state=init)
    assert_abs(y, g["y"], name + " y", 2e-4)
    assert_abs(fs, g["final_states"], name + " final_states", 2e-5)


def test_ssd_ragged_output_equals_recurrence(golden_dir):
    # seqlen % chunk != 0: the reference pads dt BEFORE softplus, which over-decays final_states but leaves y intact
    g = load(golden_dir, "ssd_ragged_len")
    y, _ = orc.ssd_recurrence(g["x"], g["dt"], g["A"], g["B"], g["C"], D=g["D"], dt_bias=g["dt_bias"])
    assert_abs(y, g["y"], "ragged y", 2e-4)


def test_conv_update_reproduces_prefill_columns():
    r = np.random.default_rng(1)
    B, D, S, W = 2, 11, 9, 4
    x = r.standard_normal((B, D, S), np.float32)
    w = r.standard_normal((D, W), np.float32)
    b = r.standard_normal(D).astype(np.float32)
    full = orc.causal_conv1d(x, w, b)
    st = np.zeros((B, D, W - 1), np.float32)
    for t in range(S):
        y = orc.causal_conv1d_update(np.ascontiguousarray(x[:, :, t]), st, w, b)
        assert np.array_equal(y, full[:, :, t])
    assert np.array_equal(st, x[:, :, S - 3:])


def _cfg0_inputs():
    cfg = synth.CONFIGS["cfg0"]
    return cfg, synth.make_weights(cfg, 0), synth.make_input(cfg, 0)


def test_mixer_cfg0_matches_reference_composition(golden_dir):
    g = load(golden_dir, "mixer_cfg0")
    cfg, w, u = _cfg0_inputs()
    chk = np.array([np.float64(np.abs(v).sum()) for v in [u] + [w[k] for k in sorted(w)]])
    assert np.allclose(chk, g["input_checksums"], rtol=0, atol=0), "seeded input generator drifted from the golden file"
    res = orc.mixer_prefill(u, w, cfg, want_intermediates=True)
    assert np.array_equal(res["zxbcdt"], g["zxbcdt"])
    assert_abs(res["y"], g["y"], "y", 2e-4)
    assert_abs(res["g"], g["g"], "g", 1e-3)
    assert_abs(res["out"], g["out"], "out", 1e-3)
    assert_abs(res["final_state"], g["final_states"], "final_states", 2e-5)


def test_mixer_decode_continues_prefill():
    cfg, w, _ = _cfg0_inputs()
    u = synth.make_input(cfg, 0, batch=2, seqlen=40)
    # prefill 32 tokens (one chunk), then decode 8 tokens == prefill of all 40 with the recurrence as the scan
    head = orc.mixer_prefill(u[:, :32], w, cfg)
    cs, ss = head["conv_state"].copy(), head["final_state"].copy()
    outs = [orc.mixer_decode(np.ascontiguousarray(u[:, 32 + t]), w, cfg, cs, ss) for t in range(8)]
    cfg64 = dict(cfg, chunk=8)  # 40 = 5 chunks of 8, so the chunked scan sees no padding
    full = orc.mixer_prefill(u, w, cfg64)
    assert_abs(np.stack(outs, 1), full["out"][:, 32:], "decode vs prefill", 1e-3)
    assert_abs(ss, full["final_state"], "ssm_state", 2e-5)


def test_rms_norm_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "rms_norm.npz"))
    y = orc.rms_norm(g["x"], g["w"], float(g["eps"]))
    assert np.array_equal(y, g["y_ref"])          # the reference's compiled tensor_rms_norm<float32, CPU>: bit-exact
    assert_abs(y, g["y_torch"], "rms_norm vs torch", 1e-5)
    yz = orc.rms_norm(g["x"], g["w"], float(g["eps"]), zero_centered=True)
    assert_abs(yz, orc.rms_norm(g["x"], g["w"] + 1.0, float(g["eps"])), "zero-centered weight", 1e-5)


def test_decoder_layer_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "decoder_cfg0.npz"))
    cfg = synth.CONFIGS["cfg0"]
    w, hidden = synth.make_weights(cfg, 0), synth.make_input(cfg, 0)
    got = orc.decoder_prefill(hidden, w, g["input_norm_weight"], float(g["rms_eps"]), cfg)
    assert np.array_equal(orc.rms_norm(hidden, g["input_norm_weight"], float(g["rms_eps"])), g["normed"])
    assert_abs(got["out"], g["out"], "decoder layer out", 1e-3)
    assert_abs(got["final_state"], g["final_states"], "decoder layer final state", 1e-4)


def test_reference_build_agrees_when_present():
    if orc.ref_lib() is None:
        pytest.skip("reference CPU operators not built in this checkout (oracle/_ref)")
    r = np.random.default_rng(3)
    x = r.standard_normal((2, 7, 19), np.float32)
    w = r.standard_normal((7, 4), np.float32)
    b = r.standard_normal(7).astype(np.float32)
    assert np.array_equal(orc.causal_conv1d(x, w, b), orc.ref_causal_conv1d(x, w, b))
    a, z = r.standard_normal((4, 40), np.float32), r.standard_normal((4, 40), np.float32)
    nw = r.standard_normal(40).astype(np.float32)
    assert np.array_equal(orc.gated_rmsnorm(a, z, nw, 1e-5), orc.ref_gated_rmsnorm(a, z, nw, 1e-5))
    m, k = r.standard_normal((6, 50), np.float32), r.standard_normal((50, 9), np.float32)
    assert np.array_equal(orc.linear(m, k), orc.ref_linear(m, k))
    assert np.array_equal(orc.rms_norm(a, nw, 1e-5), orc.ref_rms_norm(a, nw, 1e-5))


def test_threads_do_not_change_results():
    cfg, w, u = _cfg0_inputs()
    a = orc.mixer_prefill(u, w, cfg)["out"]
    orc.set_num_threads(4)
    try:
        b = orc.mixer_prefill(u, w, cfg)["out"]
    finally:
        orc.set_num_threads(1)
    assert np.array_equal(a, b)
