"""World-size-2 gloo test (CPU) of the multi-GPU host logic: batch sharding and the max-over-ranks timing reduction."""
import os
import socket

import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp  # noqa: E402

from anygpu_b200 import dist as bdist  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = bdist.shard_bounds(7, world, rank)
    slowest = bdist.max_over_ranks(0.5 + rank)           # rank 1 is the slow one
    tput = bdist.job_throughput((hi - lo) * 100, 0.5 + rank)
    dist.barrier()
    out.put((rank, lo, hi, slowest, tput))
    dist.destroy_process_group()


def test_two_rank_sharding_and_timing_reduction():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, lo0, hi0, s0, t0), (r1, lo1, hi1, s1, t1) = res
    assert (lo0, hi0, lo1, hi1) == (0, 4, 4, 7)          # contiguous, disjoint, covering
    assert s0 == s1 == 1.5                                # both ranks see the slowest rank's time
    assert t0 == t1 == pytest.approx(700 / 1.5)           # whole-job units / slowest time


def test_shard_bounds_properties():
    for batch in (1, 4, 32, 33):
        for world in (1, 2, 4, 8):
            spans = [bdist.shard_bounds(batch, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_single_process_is_identity():
    assert bdist.max_over_ranks(3.25) == 3.25
    assert bdist.job_throughput(10, 2.0) == 5.0


def test_sequence_parallel_segment_bounds():
    from anygpu_b200.dist import sp_segments
    assert sp_segments(4096, 4) == [(0, 1024), (1024, 2048), (2048, 3072), (3072, 4096)]
    assert sp_segments(1000, 4, align=256) == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    assert sp_segments(300, 4, align=256) == [(0, 256), (256, 300), (300, 300), (300, 300)]
    for seqlen, world, align in [(777, 3, 1), (4097, 8, 256), (5, 8, 1)]:
        segs = sp_segments(seqlen, world, align)
        assert segs[0][0] == 0 and segs[-1][1] == seqlen and all(a[1] == b[0] for a, b in zip(segs, segs[1:]))
