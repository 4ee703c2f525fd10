"""Host-side pieces of bench.py that need no GPU: the pipeline schedule of the head-sharded runs."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_tp_chunk_schedule_covers_the_batch_once():
    for batch in (1, 2, 7, 8, 32):
        for world in (1, 2, 4, 8):
            for chunk in (0, 1, 2, 3, 8, 64):
                sched = bench.tp_chunk_schedule(batch, world, chunk)
                assert sum(sched) == batch and all(v > 0 for v in sched), (batch, world, chunk, sched)
                want = chunk if chunk > 0 else max(2, world)
                assert max(sched) == min(want, batch), (batch, world, chunk, sched)
    assert bench.tp_chunk_schedule(32, 8, 0) == [8, 8, 8, 8]
    assert bench.tp_chunk_schedule(32, 2, 0) == [2] * 16

