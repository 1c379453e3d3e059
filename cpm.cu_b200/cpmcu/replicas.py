"""Request replicas: the unit of work of this path is one request (batch 1, one KV
cache, one tree) and nothing below it shards, so N GPUs run N independent
processes with their own weights and prompts.  The only cross-rank step is the
bookkeeping here: total tokens and the slowest rank's time."""
import torch


def combine_ranks(tokens, device_seconds, wall_seconds, dist=None, device="cpu"):
    """Aggregate one measurement over all ranks: (sum of tokens, max device time, max wall time).
    `dist` is torch.distributed (initialised) or None for a single process."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(tokens), float(device_seconds), float(wall_seconds)
    tok = torch.tensor([float(tokens)], dtype=torch.float64, device=device)
    tim = torch.tensor([float(device_seconds), float(wall_seconds)], dtype=torch.float64, device=device)
    dist.all_reduce(tok, op=dist.ReduceOp.SUM)
    dist.all_reduce(tim, op=dist.ReduceOp.MAX)
    return float(tok[0]), float(tim[0]), float(tim[1])


def replica_seed(base_seed, rank):
    """Distinct prompt seed per replica."""
    return int(base_seed) + int(rank)
