"""GPU parity tests of the whole Mamba2 mixer through the C ABI (prefill, decode, prefill -> decode hand-off).

Gate: per-operator parity with zero elements outside tolerance lives in test_gpu_ops.py. End to end, the f16 mixer is
compared with the oracle that rounds to binary16 at the same operator boundaries (what a chain of Tensor<float16>
operators does). At the sizes of this file every end-to-end comparison measures ZERO elements outside rel 2e-2 / abs 2e-3
(the session prints the measured figures), so zero is what the assertions allow; the reference's global rel-L2 metric
(tests/test_tools.hpp:77-103, threshold 1e-2) is additionally required to stay below 2e-3 (3e-3 for decode chains)."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from anygpu_b200 import synth  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from tolerance import assert_abs, assert_close_f16, rel_l2  # noqa: E402

pytestmark = pytest.mark.gpu

SMALL = dict(batch=2, seqlen=512, d_model=256, d_inner=512, nheads=8, headdim=64, d_state=64, ngroups=1, d_conv=4, chunk=256,
             eps=1e-5)
SMALL_G2 = dict(batch=1, seqlen=256, d_model=128, d_inner=512, nheads=8, headdim=64, d_state=64, ngroups=2, d_conv=4, chunk=128,
                eps=1e-5, norm_group_size=256)


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from anygpu_b200 import ops as _ops
    return _ops


def f16w(w):
    return {k: (synth.to_f16_values(v) if k not in ("dt_bias", "A_log", "D") else v) for k, v in w.items()}


def host(t):
    return t.float().cpu().numpy()


def test_mixer_cfg0_fp32_matches_reference_composition(ops, golden_dir):
    g = np.load(os.path.join(golden_dir, "mixer_cfg0.npz"))
    cfg = synth.CONFIGS["cfg0"]
    w, u = synth.make_weights(cfg, 0), synth.make_input(cfg, 0)
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float32))
    cache = ops.ZambaMambaCache.zeros(cfg, cfg["batch"], torch.float32)
    out = mixer.prefill(torch.from_numpy(u).cuda(), cache)
    # every stage of the golden was produced by reference code; its fp32 comparisons use abs 1e-3
    assert_abs(host(out), g["out"], "mixer out", 1e-3)
    assert_abs(host(cache.ssm_state), g["final_states"], "final ssm state", 1e-4)


@pytest.mark.parametrize("cfg", [SMALL, SMALL_G2], ids=["g1", "g2_grouped_norm"])
@pytest.mark.parametrize("layout", ["KN", "NK"])
def test_mixer_prefill_f16(ops, cfg, layout):
    w = f16w(synth.make_weights(cfg, 1))
    u = synth.to_f16_values(synth.make_input(cfg, 1))
    want = orc.mixer_prefill(u, w, cfg, f16io=True)
    pure = orc.mixer_prefill(u, w, cfg, f16io=False)
    wt = ops.ZambaMamba2weights.from_numpy(w, torch.float16, layout=ops.W_KN if layout == "KN" else ops.W_NK)
    mixer = ops.Mamba2Mixer(cfg, wt)
    cache = ops.ZambaMambaCache.zeros(cfg, cfg["batch"], torch.float16)
    out = host(mixer.prefill(torch.from_numpy(u).cuda().half(), cache))
    assert_close_f16(out, want["out"], "mixer out vs op-boundary-rounded oracle")
    assert rel_l2(out, want["out"]) < 2e-3
    assert rel_l2(out, pure["out"]) < 2e-3  # against the pure-fp32 oracle as well
    assert_close_f16(host(cache.ssm_state), want["final_state"], "final ssm state")
    assert_close_f16(host(cache.conv_state), want["conv_state"], "conv state")


@pytest.mark.parametrize("nheads,d_state", [(4, 64), (3, 16), (12, 64)])
def test_mixer_f16_head_counts_off_the_8_element_grid(ops, nheads, d_state):
    """d_in_proj = 2 d_inner + 2 G N + nheads is a multiple of 8 only when nheads is: with 4, 3 or 12 heads the projection
    runs on the SIMT GEMM and the in_proj output keeps a padded row stride inside the workspace. Prefill, states and a decode
    step against the oracle."""
    cfg = dict(batch=2, seqlen=200, d_model=128, d_inner=nheads * 64, nheads=nheads, headdim=64, d_state=d_state, ngroups=1, d_conv=4,
               chunk=64, eps=1e-5)
    assert (2 * cfg["d_inner"] + 2 * d_state + nheads) % 8 != 0
    w = f16w(synth.make_weights(cfg, 21))
    u = synth.to_f16_values(synth.make_input(cfg, 21, batch=2, seqlen=201))
    want = orc.mixer_prefill(u[:, :200], w, dict(cfg, chunk=8), f16io=True)  # 200 = 25 chunks of 8: no padding in the oracle
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float16))
    cache = ops.ZambaMambaCache.zeros(cfg, 2, torch.float16)
    ud = torch.from_numpy(u).cuda().half()
    out = host(mixer.prefill(ud[:, :200].contiguous(), cache))
    assert_close_f16(out, want["out"], f"mixer out, {nheads} heads")
    assert_close_f16(host(cache.ssm_state), want["final_state"], "final ssm state")
    assert_close_f16(host(cache.conv_state), want["conv_state"], "conv state")
    ocs, oss = want["conv_state"].copy(), want["final_state"].copy()
    got = host(mixer.decode(ud[:, 200].contiguous(), cache))
    wd = orc.mixer_decode(np.ascontiguousarray(u[:, 200]), w, cfg, ocs, oss, f16io=True)
    assert_close_f16(got, wd, f"decode step, {nheads} heads")


def test_mixer_prefill_host_call_equals_device_call(ops):
    cfg = SMALL
    w = f16w(synth.make_weights(cfg, 2))
    u = torch.from_numpy(synth.make_input(cfg, 2)).half()
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float16))
    dev_out = mixer.prefill(u.cuda()).cpu()
    u_pin, out_pin = u.pin_memory(), torch.empty_like(u).pin_memory()
    mixer.prefill_host(u_pin, out_pin)
    torch.cuda.synchronize()
    assert torch.equal(dev_out, out_pin)


def test_stage_timing_windows_plain_and_inside_a_captured_graph(ops):
    """b200_stage_timing_*: every stage of every call (mode 1), in_proj of every fourth call only (mode 2), and calls that were
    captured into a CUDA graph, whose events are recorded when the graph is replayed."""
    import ctypes
    from anygpu_b200 import capi
    lib = capi.load()
    cfg = SMALL
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(f16w(synth.make_weights(cfg, 2)), torch.float16))
    u = torch.from_numpy(synth.to_f16_values(synth.make_input(cfg, 2))).cuda().half()
    out = torch.empty_like(u)
    want = mixer.prefill(u).clone()
    ms, calls = (ctypes.c_float * 5)(), ctypes.c_int(0)
    try:
        assert lib.b200_stage_timing_enable(1) == 0
        for _ in range(3):
            mixer.prefill(u, out=out)
        assert lib.b200_stage_timing_collect(ms, ctypes.byref(calls)) == 0
        assert calls.value == 3 and all(0.0 < v < 50.0 for v in ms), (calls.value, list(ms))
        assert lib.b200_stage_timing_enable(2) == 0
        for _ in range(8):
            mixer.prefill(u, out=out)
        assert lib.b200_stage_timing_collect(ms, ctypes.byref(calls)) == 0
        assert calls.value == 2 and ms[0] > 0.0 and all(v == 0.0 for v in list(ms)[1:]), (calls.value, list(ms))
        assert lib.b200_stage_timing_enable(1) == 0
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            mixer.prefill(u, out=out)
            mixer.prefill(u, out=out)
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert lib.b200_stage_timing_collect(ms, ctypes.byref(calls)) == 0
        assert calls.value == 2 and all(0.0 < v < 50.0 for v in ms), (calls.value, list(ms))
        assert torch.equal(out, want)
    finally:
        lib.b200_stage_timing_enable(0)


def test_back_to_back_host_calls_with_ready_inputs_overlap_and_stay_correct(ops):
    """B200_HOST_OVERLAP: consecutive calls on one workspace and stream run their copy-in under the call before them.
    Six calls with different inputs and outputs queued without a synchronisation in between, then one call of another shape
    (which must fall back to the ordered form), every output equal to the device call's bit for bit. The last call feeds on the
    output of the one before it WITHOUT the flag, so it has to wait for that copy-out."""
    cfg = SMALL
    w = f16w(synth.make_weights(cfg, 2))
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float16))
    us = [torch.from_numpy(synth.make_input(cfg, 40 + i)).half() for i in range(6)]
    want = [mixer.prefill(u.cuda()).cpu() for u in us]
    pins = [u.pin_memory() for u in us]
    outs = [torch.zeros_like(u).pin_memory() for u in us]
    for u, o in zip(pins, outs):
        mixer.prefill_host(u, o, overlap=True)
    short = torch.from_numpy(synth.make_input(cfg, 50, batch=1, seqlen=100)).half()
    short_pin, short_out = short.pin_memory(), torch.zeros_like(short).pin_memory()
    mixer.prefill_host(short_pin, short_out, overlap=True)
    chained = torch.zeros_like(short).pin_memory()
    mixer.prefill_host(short_out, chained)  # input produced by the call before: ordered on the stream
    torch.cuda.synchronize()
    for i in range(6):
        assert torch.equal(outs[i], want[i]), i
    assert torch.equal(short_out, mixer.prefill(short.cuda()).cpu())
    assert torch.equal(chained, mixer.prefill(short_out.cuda()).cpu())


@pytest.mark.parametrize("dtype", ["f16", "f16_nk", "f32"])
def test_mixer_decode_steps(ops, dtype):
    cfg = dict(SMALL, batch=5)
    layout = ops.W_NK if dtype == "f16_nk" else ops.W_KN
    dtype = dtype[:3]
    td = torch.float16 if dtype == "f16" else torch.float32
    w = synth.make_weights(cfg, 3)
    cs, ss = synth.make_decode_state(cfg, 3)
    us = synth.make_input(cfg, 3, batch=5, seqlen=6)
    if dtype == "f16":
        w, cs, us = f16w(w), synth.to_f16_values(cs), synth.to_f16_values(us)
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, td, layout=layout))
    cache = ops.ZambaMambaCache(torch.from_numpy(cs).cuda().to(td), torch.from_numpy(ss).cuda())
    ocs, oss = cs.copy(), ss.copy()
    for t in range(us.shape[1]):
        got = host(mixer.decode(torch.from_numpy(np.ascontiguousarray(us[:, t])).cuda().to(td), cache))
        want = orc.mixer_decode(np.ascontiguousarray(us[:, t]), w, cfg, ocs, oss, f16io=(dtype == "f16"))
        if dtype == "f16":
            assert_close_f16(got, want, f"decode step {t}")
            assert rel_l2(got, want) < 2e-3
        else:
            assert_abs(got, want, f"decode step {t}", 1e-3)
    assert_abs(host(cache.ssm_state), oss, "ssm state after decode", 2e-3)
    assert_close_f16(host(cache.conv_state), ocs, "conv state after decode")


def test_decode_replayed_from_a_cuda_graph_equals_eager_decode(ops):
    cfg = dict(SMALL, batch=3)
    w = f16w(synth.make_weights(cfg, 7))
    cs, ss = synth.make_decode_state(cfg, 7)
    us = torch.from_numpy(synth.make_input(cfg, 7, batch=3, seqlen=4)).cuda().half()
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float16))
    mk = lambda: ops.ZambaMambaCache(torch.from_numpy(cs).cuda().half(), torch.from_numpy(ss).cuda())
    eager_cache, graph_cache = mk(), mk()
    u_buf, o_buf = torch.empty_like(us[:, 0]), torch.empty_like(us[:, 0])
    u_buf.copy_(us[:, 0])
    graph = mixer.capture_decode(u_buf, graph_cache, o_buf)
    assert torch.equal(graph_cache.ssm_state, eager_cache.ssm_state)  # capturing does not advance the cache
    for t in range(us.shape[1]):
        want = mixer.decode(us[:, t].contiguous(), eager_cache).clone()
        u_buf.copy_(us[:, t])
        graph.replay()
        assert torch.equal(o_buf, want), t
    assert torch.equal(graph_cache.ssm_state, eager_cache.ssm_state)
    assert torch.equal(graph_cache.conv_state, eager_cache.conv_state)


def test_several_decode_steps_in_one_cuda_graph_equal_eager_steps(ops):
    cfg = dict(SMALL, batch=3)
    w = f16w(synth.make_weights(cfg, 9))
    cs, ss = synth.make_decode_state(cfg, 9)
    us = torch.from_numpy(synth.make_input(cfg, 9, batch=3, seqlen=6)).cuda().half().transpose(0, 1).contiguous()  # (steps, b, d)
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float16))
    mk = lambda: ops.ZambaMambaCache(torch.from_numpy(cs).cuda().half(), torch.from_numpy(ss).cuda())
    eager_cache, graph_cache = mk(), mk()
    outs = torch.empty_like(us)
    graph = mixer.capture_decode_steps(us, graph_cache, outs)
    assert torch.equal(graph_cache.ssm_state, eager_cache.ssm_state)  # capturing does not advance the cache
    graph.replay()
    torch.cuda.synchronize()
    for t in range(us.shape[0]):
        want = mixer.decode(us[t], eager_cache)
        assert torch.equal(outs[t], want), t
    assert torch.equal(graph_cache.ssm_state, eager_cache.ssm_state)
    assert torch.equal(graph_cache.conv_state, eager_cache.conv_state)


def test_prefill_then_decode_continues_the_sequence(ops):
    cfg = dict(SMALL, batch=2, chunk=64)
    w = f16w(synth.make_weights(cfg, 4))
    u = synth.to_f16_values(synth.make_input(cfg, 4, batch=2, seqlen=128 + 8))
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float16))
    cache = ops.ZambaMambaCache.zeros(cfg, 2, torch.float16)
    ud = torch.from_numpy(u).cuda().half()
    mixer.prefill(ud[:, :128].contiguous(), cache)
    outs = [host(mixer.decode(ud[:, 128 + t].contiguous(), cache)) for t in range(8)]
    full = orc.mixer_prefill(u, w, dict(cfg, chunk=8), f16io=True)  # 136 = 17 chunks of 8: no padding in the oracle
    got = np.stack(outs, axis=1)
    assert_close_f16(got, full["out"][:, 128:], "decode continues prefill")
    assert rel_l2(got, full["out"][:, 128:]) < 3e-3


@pytest.mark.parametrize("tp", [2, 4])
def test_head_sharded_tp_ranks_emulated_on_one_gpu(ops, tp):
    """Tensor parallelism without a second GPU: the ranks run one after the other on this device and their partial outputs
    and partial sums of squares are added by hand (what the all-reduce does). The result must match the unsharded mixer."""
    cfg = dict(SMALL, nheads=8, ngroups=2, d_state=64, seqlen=256, chunk=128, batch=2)
    w = f16w(synth.make_weights(cfg, 6))
    u = synth.to_f16_values(synth.make_input(cfg, 6))
    want = orc.mixer_prefill(u, w, cfg, f16io=True)["out"]
    ud = torch.from_numpy(u).cuda().half()
    whole = host(ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float16)).prefill(ud))
    loc = synth.tp_local_config(cfg, tp)
    out_sum = torch.zeros(cfg["batch"], cfg["seqlen"], cfg["d_model"], device="cuda", dtype=torch.float32)
    ss_sum = torch.zeros(cfg["batch"] * cfg["seqlen"], device="cuda")
    last = None
    for r in range(tp):
        wl = ops.ZambaMamba2weights.from_numpy(synth.shard_weights_tp(w, cfg, tp, r), torch.float16)
        last = ops.Mamba2MixerTP(loc, wl, cfg["d_inner"])
        po, ss = last.partial(ud)
        out_sum += po.float()
        ss_sum += ss
    got = host(last.finish(out_sum.half(), ss_sum))
    assert_close_f16(got, want, f"tp{tp} vs oracle")
    assert rel_l2(got, want) < 2e-3
    assert rel_l2(got, whole) < 2e-3


def test_decoder_layer_cfg0_fp32_matches_reference_composition(ops, golden_dir):
    g = np.load(os.path.join(golden_dir, "decoder_cfg0.npz"))
    cfg = synth.CONFIGS["cfg0"]
    w, hidden = synth.make_weights(cfg, 0), synth.make_input(cfg, 0)
    layer = ops.Mamba2DecoderLayer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float32),
                                   torch.from_numpy(g["input_norm_weight"]).cuda(), float(g["rms_eps"]))
    cache = ops.ZambaMambaCache.zeros(cfg, cfg["batch"], torch.float32)
    out = layer.prefill(torch.from_numpy(hidden).cuda(), cache)
    assert_abs(host(out), g["out"], "decoder layer out (every golden stage produced by reference code)", 1e-3)
    assert_abs(host(cache.ssm_state), g["final_states"], "final ssm state", 1e-4)


@pytest.mark.parametrize("layout", ["KN", "NK"])
def test_decoder_layer_f16_prefill_then_decode(ops, layout):
    cfg = dict(SMALL, batch=3, seqlen=256)
    w = f16w(synth.make_weights(cfg, 8))
    w_in = synth.to_f16_values(1.0 + 0.1 * np.random.default_rng(8).standard_normal(cfg["d_model"]).astype(np.float32))
    h = synth.to_f16_values(synth.make_input(cfg, 8, batch=3, seqlen=256 + 4))
    wt = ops.ZambaMamba2weights.from_numpy(w, torch.float16, layout=ops.W_KN if layout == "KN" else ops.W_NK)
    layer = ops.Mamba2DecoderLayer(cfg, wt, torch.from_numpy(w_in).cuda().half(), 1e-5)
    cache = ops.ZambaMambaCache.zeros(cfg, 3, torch.float16)
    hd = torch.from_numpy(h).cuda().half()
    want = orc.decoder_prefill(h[:, :256], w, w_in, 1e-5, cfg, f16io=True)
    out = host(layer.prefill(hd[:, :256].contiguous(), cache))
    assert_close_f16(out, want["out"], "decoder layer prefill")
    assert rel_l2(out, want["out"]) < 2e-3
    # in place: the residual stream is overwritten by the layer's output
    buf = hd[:, :256].contiguous()
    layer.prefill(buf, out=buf)
    assert torch.equal(buf.float().cpu(), torch.from_numpy(out))
    ocs, oss = want["conv_state"].copy(), want["final_state"].copy()
    for t in range(4):
        ht = np.ascontiguousarray(h[:, 256 + t])
        got = host(layer.decode(hd[:, 256 + t].contiguous(), cache))
        wd = orc.decoder_decode(ht, w, w_in, 1e-5, cfg, ocs, oss, f16io=True)
        assert_close_f16(got, wd, f"decoder layer decode step {t}")
        assert rel_l2(got, wd) < 3e-3


@pytest.mark.parametrize("pieces", [(512,), (256, 256), (100, 7, 300, 105), (1, 511)])
def test_prefill_in_pieces_equals_one_prefill(ops, pieces):
    """Chunked prefill: any split of the prompt gives the same outputs and states (piece lengths need not be multiples of
    the scan chunk); a decode step continues from the cache afterwards."""
    cfg = dict(SMALL, batch=2, seqlen=512, chunk=128)
    w = f16w(synth.make_weights(cfg, 10))
    u = synth.to_f16_values(synth.make_input(cfg, 10, batch=2, seqlen=513))
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float16))
    ud = torch.from_numpy(u).cuda().half()
    whole_cache = ops.ZambaMambaCache.zeros(cfg, 2, torch.float16)
    whole = mixer.prefill(ud[:, :512].contiguous(), whole_cache)
    cache = ops.ZambaMambaCache.zeros(cfg, 2, torch.float16)
    outs, t0 = [], 0
    for n in pieces:
        outs.append(mixer.prefill_continue(ud[:, t0:t0 + n].contiguous(), cache))
        t0 += n
    got = torch.cat(outs, dim=1)
    want = orc.mixer_prefill(u[:, :512], w, dict(cfg, chunk=8), f16io=True)  # 512 = 64 chunks of 8: no padding in the oracle
    assert_close_f16(host(got), want["out"], f"pieces {pieces} vs oracle")
    assert rel_l2(host(got), want["out"]) < 2e-3
    assert rel_l2(host(got), host(whole)) < 2e-3
    assert torch.equal(cache.conv_state, whole_cache.conv_state)  # the last three inputs, whatever the split
    assert_close_f16(host(cache.ssm_state), want["final_state"], "ssm state after the pieces")
    d1 = mixer.decode(ud[:, 512].contiguous(), cache)
    d2 = mixer.decode(ud[:, 512].contiguous(), whole_cache)
    assert rel_l2(host(d1), host(d2)) < 3e-3


@pytest.mark.parametrize("lens", [[512, 100, 0, 1, 257, 3], [128, 128], [0], [700]])
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_packed_variable_length_batch_equals_separate_prefills(ops, lens, dtype):
    """cu_seqlens batches: every sequence of the packed call gets the outputs and final states of a prefill of that sequence
    alone (bit for bit: same kernels on the same rows), nothing leaks across a boundary, an empty sequence hands on its
    initial state; one sequence is also checked against the oracle."""
    cfg = dict(SMALL, batch=1, seqlen=max(max(lens), 1), chunk=128)
    td = torch.float16 if dtype == "f16" else torch.float32
    w = synth.make_weights(cfg, 12)
    total = sum(lens)
    u = synth.make_input(cfg, 12, batch=1, seqlen=max(total, 1))[0, :total]
    if dtype == "f16":
        w, u = f16w(w), synth.to_f16_values(u)
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, td))
    ud = torch.from_numpy(np.ascontiguousarray(u)).cuda().to(td)
    nseq = len(lens)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    H, P, N = cfg["nheads"], cfg["headdim"], cfg["d_state"]
    init = (torch.randn(nseq, H, P, N, device="cuda", generator=torch.Generator("cuda").manual_seed(3)) * 0.1).contiguous()
    cache = ops.ZambaMambaCache.zeros(cfg, nseq, td)
    cache.conv_state.fill_(7.0)  # must be overwritten for every sequence
    got = mixer.prefill_varlen(ud, cu, initial_states=init, cache=cache)
    assert got.shape == ud.shape
    for s, n in enumerate(lens):
        one = ops.ZambaMambaCache.zeros(cfg, 1, td)
        if n == 0:
            assert torch.equal(cache.ssm_state[s], init[s])
            assert torch.count_nonzero(cache.conv_state[s]) == 0
            continue
        alone = mixer.prefill(ud[cu[s]:cu[s + 1]].unsqueeze(0).contiguous(), one, initial_states=init[s:s + 1].contiguous())
        assert torch.equal(got[cu[s]:cu[s + 1]], alone[0]), f"sequence {s} of lengths {lens}"
        assert torch.equal(cache.ssm_state[s], one.ssm_state[0])
        assert torch.equal(cache.conv_state[s], one.conv_state[0])
    s = int(np.argmax(lens))
    if lens[s] > 0 and lens[s] % 4 == 0:
        want = orc.mixer_prefill(u[None, cu[s]:cu[s + 1]], w, dict(cfg, chunk=4), f16io=dtype == "f16",
                                 initial_states=host(init[s:s + 1]))
        if dtype == "f16":
            assert_close_f16(host(got[cu[s]:cu[s + 1]])[None], want["out"], "packed sequence vs oracle")
        assert rel_l2(host(got[cu[s]:cu[s + 1]])[None], want["out"]) < (2e-3 if dtype == "f16" else 1e-4)


def test_packed_batch_of_many_short_sequences(ops, monkeypatch):
    """256 sequences of 20 to 44 tokens (and a few empty ones) in one packed call: every sequence equals a prefill of it alone
    bit for bit, states included, and one of them is checked against the oracle. The packed call is a fixed handful of launches
    (with the scan left to choose its kernel: B200_SSD_FUSED=0 sends this batch through the per-sequence loop)."""
    from anygpu_b200 import capi
    monkeypatch.delenv("B200_SSD_FUSED", raising=False)
    cfg = dict(SMALL, batch=1, seqlen=64, chunk=128)
    r = np.random.default_rng(5)
    lens = [int(v) for v in r.integers(20, 45, 256)]
    for i in (7, 100, 255):
        lens[i] = 0
    total = sum(lens)
    w = f16w(synth.make_weights(cfg, 14))
    u = synth.to_f16_values(synth.make_input(cfg, 14, batch=1, seqlen=total)[0])
    mixer = ops.Mamba2Mixer(cfg, ops.ZambaMamba2weights.from_numpy(w, torch.float16))
    ud = torch.from_numpy(np.ascontiguousarray(u)).cuda().half()
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    H, P, N = cfg["nheads"], cfg["headdim"], cfg["d_state"]
    init = (torch.randn(len(lens), H, P, N, device="cuda", generator=torch.Generator("cuda").manual_seed(4)) * 0.1).contiguous()
    cache = ops.ZambaMambaCache.zeros(cfg, len(lens), torch.float16)
    cache.conv_state.fill_(7.0)
    lib = capi.load()
    mixer.prefill_varlen(ud, cu, initial_states=init, cache=cache)  # workspace and kernel attributes set up
    lib.b200_launch_count(1)
    got = mixer.prefill_varlen(ud, cu, initial_states=init, cache=cache)
    launches = lib.b200_launch_count(1)
    assert launches <= 6, launches  # in_proj, conv1d + dt, scan, gated norm, out_proj
    for s in (0, 1, 7, 99, 100, 101, 254, 255):
        n = lens[s]
        if n == 0:
            assert torch.equal(cache.ssm_state[s], init[s]) and torch.count_nonzero(cache.conv_state[s]) == 0
            continue
        one = ops.ZambaMambaCache.zeros(cfg, 1, torch.float16)
        alone = mixer.prefill(ud[cu[s]:cu[s + 1]].unsqueeze(0).contiguous(), one, initial_states=init[s:s + 1].contiguous())
        assert torch.equal(got[cu[s]:cu[s + 1]], alone[0]), s
        assert torch.equal(cache.ssm_state[s], one.ssm_state[0]) and torch.equal(cache.conv_state[s], one.conv_state[0]), s
    s = 33
    want = orc.mixer_prefill(u[None, cu[s]:cu[s + 1]], w, dict(cfg, chunk=lens[s]), f16io=True, initial_states=host(init[s:s + 1]))
    assert_close_f16(host(got[cu[s]:cu[s + 1]])[None], want["out"], "one of 256 packed sequences vs oracle")
    assert_close_f16(host(cache.ssm_state[s:s + 1]), want["final_state"], "its final state")


@pytest.mark.parametrize("bounds", [[0, 128, 256, 384, 512], [0, 100, 101, 300, 512], [0, 512]])
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_sequence_parallel_segments_emulated_on_one_gpu(ops, bounds, dtype):
    """Sequence parallelism without a second GPU: the segments run one after the other on this device, the gathered
    per-segment states are what the all-gather would deliver. Outputs and final states must equal one prefill of the whole
    sequence (any segment lengths, aligned to the chunk or not)."""
    cfg = dict(SMALL, batch=2, seqlen=512, chunk=128)
    td = torch.float16 if dtype == "f16" else torch.float32
    w = synth.make_weights(cfg, 11)
    u = synth.make_input(cfg, 11)
    if dtype == "f16":
        w, u = f16w(w), synth.to_f16_values(u)
    wt = ops.ZambaMamba2weights.from_numpy(w, td)
    ud = torch.from_numpy(u).cuda().to(td)
    whole_cache = ops.ZambaMambaCache.zeros(cfg, 2, td)
    whole = ops.Mamba2Mixer(cfg, wt).prefill(ud, whole_cache)
    R = len(bounds) - 1
    ranks = [ops.Mamba2MixerSP(cfg, wt) for _ in range(R)]
    caches = [ops.ZambaMambaCache.zeros(cfg, 2, td) for _ in range(R)]
    states, decays = [], []
    for r in range(R):
        lo, hi = bounds[r], bounds[r + 1]
        halo = ud[:, lo - 3:lo].contiguous() if r > 0 else None
        s_, d_ = ranks[r].begin(ud[:, lo:hi].contiguous(), halo, caches[r])
        states.append(s_)
        decays.append(d_)
    gs, gd = torch.stack(states).contiguous(), torch.stack(decays).contiguous()  # what the all-gather delivers
    outs = [ranks[r].finish(ranks[r].prefix(gs, gd, r), cache=caches[r]) for r in range(R)]
    got = torch.cat(outs, dim=1)
    if dtype == "f16":
        want = orc.mixer_prefill(u, w, dict(cfg, chunk=8), f16io=True)
        assert_close_f16(host(got), want["out"], "segments vs oracle")
        assert rel_l2(host(got), host(whole)) < 2e-3
        assert_close_f16(host(caches[-1].ssm_state), want["final_state"], "final state on the last rank")
    else:
        want = orc.mixer_prefill(u, w, dict(cfg, chunk=8))
        assert_abs(host(got), want["out"], "segments vs oracle", 1e-3)
        assert_abs(host(caches[-1].ssm_state), want["final_state"], "final state on the last rank", 1e-4)
    assert torch.equal(caches[-1].conv_state, whole_cache.conv_state)
