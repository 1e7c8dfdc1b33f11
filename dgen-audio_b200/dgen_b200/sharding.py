"""Voice sharding across the GPUs of one box (one process per GPU, torch.distributed).

The render path has no cross-voice dependency: `spectralLossFFTBatched` sums per voice and then takes a
batch mean (Sources/DGen/Emit+SpectralLoss.swift:889-938), so each rank renders and scores its own
voices; only scalar losses (and, in training, controller-parameter gradients) are combined.
"""
import torch
import torch.distributed as dist


def shard_range(total_voices, rank, world):
    """Contiguous, balanced [begin, end) of the voices rank `rank` owns."""
    base, rem = divmod(total_voices, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def global_mean_loss(local_loss_mean, local_voices, device="cpu"):
    """Mean over the GLOBAL batch from per-rank means: sum_r(mean_r * B_r) / sum_r(B_r).
    (The reference applies 1/B before reducing, Emit+SpectralLoss.swift:960-961.)"""
    t = torch.tensor([float(local_loss_mean) * local_voices, float(local_voices)], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t[0] / t[1])


def max_over_ranks(values, device="cpu"):
    """Element-wise max over ranks of a list of floats (device-time aggregation of a benchmark)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def world_size():
    return dist.get_world_size() if dist.is_initialized() else 1


def allreduce_sum_(flat_grad):
    """In-place sum of a flat gradient buffer over ranks (controller-parameter gradients)."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(flat_grad, op=dist.ReduceOp.SUM)
    return flat_grad


def init_ctx_comm(ctx):
    """Gives `ctx` its own NCCL communicator over the ranks of the initialised torch.distributed group:
    rank 0 creates the id, the group's object broadcast carries it (the one use of the process group)."""
    import dgen_b200
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return False
    box = [dgen_b200.comm_unique_id() if dist.get_rank() == 0 else None]
    dist.broadcast_object_list(box, src=0)
    ctx.comm_init(dist.get_world_size(), dist.get_rank(), box[0])
    return True
