"""Sequence-parallel prefill across real GPUs (runs only where at least 2 are visible): every rank holds one segment of the
sequences, the ranks all-gather their zero-state segment states and log-decays over NCCL, and the concatenated outputs must
match the oracle's prefill of the whole sequence."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

CFG = dict(batch=2, seqlen=640, d_model=256, d_inner=512, nheads=8, headdim=64, d_state=64, ngroups=1, d_conv=4, chunk=128, eps=1e-5)


def _weights():
    from anygpu_b200 import synth
    w = synth.make_weights(CFG, 12)
    return {k: (synth.to_f16_values(v) if k not in ("dt_bias", "A_log", "D") else v) for k, v in w.items()}


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from anygpu_b200 import ops, synth
    from anygpu_b200.dist import sp_segments
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    u = torch.from_numpy(synth.to_f16_values(synth.make_input(CFG, 12))).cuda().half()
    lo, hi = sp_segments(CFG["seqlen"], world, align=CFG["chunk"])[rank]  # 640 tokens over 2 ranks: 384 + 256
    mixer = ops.Mamba2MixerSP(CFG, ops.ZambaMamba2weights.from_numpy(_weights(), torch.float16))
    cache = ops.ZambaMambaCache.zeros(CFG, CFG["batch"], torch.float16)
    halo = u[:, lo - 3:lo].contiguous() if rank > 0 else None
    seg_state, seg_logdecay = mixer.begin(u[:, lo:hi].contiguous(), halo, cache)
    states = torch.empty((world,) + tuple(seg_state.shape), dtype=torch.float32, device="cuda")
    decays = torch.empty((world,) + tuple(seg_logdecay.shape), dtype=torch.float32, device="cuda")
    dist.all_gather_into_tensor(states, seg_state)
    dist.all_gather_into_tensor(decays, seg_logdecay)
    out = mixer.finish(mixer.prefix(states, decays, rank), cache=cache)
    torch.cuda.synchronize()
    q.put((rank, lo, hi, out.float().cpu().numpy(), cache.ssm_state.cpu().numpy()))
    dist.barrier()
    dist.destroy_process_group()


def test_sequence_parallel_over_nccl_matches_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from anygpu_b200 import synth
    from oracle import oracle as orc
    from tolerance import assert_close_f16, rel_l2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    u = synth.to_f16_values(synth.make_input(CFG, 12))
    want = orc.mixer_prefill(u, _weights(), dict(CFG, chunk=8), f16io=True)
    got = np.concatenate([r[3] for r in res], axis=1)
    assert res[0][1] == 0 and res[0][2] == res[1][1] and res[1][2] == CFG["seqlen"]
    assert_close_f16(got, want["out"], "sequence-parallel over NCCL vs oracle", max_fail_fraction=1e-3)
    assert rel_l2(got, want["out"]) < 2e-3
    assert_close_f16(res[1][4], want["final_state"], "final state on the last rank", max_fail_fraction=1e-4)
