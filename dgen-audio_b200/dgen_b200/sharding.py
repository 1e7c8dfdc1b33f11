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


def allreduce_sum_(flat_grad):
    """In-place sum of a flat gradient buffer over ranks (controller-parameter gradients)."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(flat_grad, op=dist.ReduceOp.SUM)
    return flat_grad
