"""Multi-GPU plumbing for the batch-sharded mixer: one process per GPU, no collective on the data path.

Sequences are independent through every stage of the mixer, so rank r of N simply owns a contiguous slice of the
batch and a full copy of the weights. The only communication is the barrier around a timed region and the
max-over-ranks reduction of its duration. Works with any torch.distributed backend (nccl on GPUs, gloo on CPU)."""
import torch
import torch.distributed as dist


def shard_bounds(global_batch, world_size, rank):
    """[lo, hi) of the sequences owned by `rank`: contiguous, disjoint, covering, sizes differ by at most one."""
    base, extra = divmod(global_batch, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def max_over_ranks(value, device="cpu"):
    """Largest `value` (float) over all ranks; identity when no process group is initialised."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value, device="cpu"):
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def job_throughput(units_this_rank, seconds_this_rank, device="cpu"):
    """Whole-job throughput: units processed by all ranks divided by the slowest rank's time."""
    return sum_over_ranks(units_this_rank, device) / max_over_ranks(seconds_this_rank, device)


def sp_segments(seqlen, world, align=1):
    """Consecutive token ranges [start, end) of a sequence split over `world` ranks for sequence-parallel prefill: as even as
    possible, every boundary but the last a multiple of `align` (segments need not be multiples of the scan chunk, but aligned
    ones avoid a padded chunk at every boundary). Ranks past the end of a short sequence get empty ranges."""
    per = -(-seqlen // world)
    per = -(-per // align) * align
    return [(min(r * per, seqlen), min((r + 1) * per, seqlen)) for r in range(world)]
