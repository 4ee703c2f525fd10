"""Head-sharded tensor parallelism across real GPUs (runs only where at least 2 are visible): every rank computes its heads,
the addends are summed with an NCCL all-reduce, and each rank's result must match the unsharded oracle."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

CFG = dict(batch=2, seqlen=256, d_model=256, d_inner=512, nheads=8, headdim=64, d_state=64, ngroups=2, d_conv=4, chunk=128, eps=1e-5)


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from anygpu_b200 import ops, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    w = synth.make_weights(CFG, 6)
    w = {k: (synth.to_f16_values(v) if k not in ("dt_bias", "A_log", "D") else v) for k, v in w.items()}
    u = synth.to_f16_values(synth.make_input(CFG, 6))
    mixer = ops.Mamba2MixerTP(synth.tp_local_config(CFG, world),
                              ops.ZambaMamba2weights.from_numpy(synth.shard_weights_tp(w, CFG, world, rank), torch.float16), CFG["d_inner"])
    po, ss = mixer.partial(torch.from_numpy(u).cuda().half())
    dist.all_reduce(po)
    dist.all_reduce(ss)
    out = mixer.finish(po, ss).float().cpu().numpy()
    torch.cuda.synchronize()
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()


def test_tp2_over_nccl_matches_oracle():
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
    outs = dict(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    w = synth.make_weights(CFG, 6)
    w = {k: (synth.to_f16_values(v) if k not in ("dt_bias", "A_log", "D") else v) for k, v in w.items()}
    want = orc.mixer_prefill(synth.to_f16_values(synth.make_input(CFG, 6)), w, CFG, f16io=True)["out"]
    assert np.array_equal(outs[0], outs[1])
    assert_close_f16(outs[0], want, "tp2 over NCCL vs oracle", max_fail_fraction=2e-4)
    assert rel_l2(outs[0], want) < 2e-3
