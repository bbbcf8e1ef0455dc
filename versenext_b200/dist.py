"""Multi-GPU plumbing: one process per GPU, requests partitioned across ranks.

The path shards by independent requests (every rank holds both models and its own slice of the
batch), so there is no collective on the data path.  `torch.distributed` is used for what remains:
a barrier, the maximum of the ranks' device times, and sums of counters.  The same helpers run on
NCCL (GPU tensors) and on gloo (CPU tensors, used by the CPU tests).

`combine_softmax_partials` is the one real exchange the path has, for a vocabulary-sharded LM head:
every rank holds per-row (max, sum exp(x - max)) of its vocabulary slice and all ranks need the
global pair (the reference has no sharded head; its `DistributedTrainer.all_reduce`,
verse_torch/training.py:2260-2266, is the only collective call it makes).
"""

from __future__ import annotations

import os
from typing import Optional, Tuple

import numpy as np


def env_world() -> Tuple[int, int, int]:
    """(world_size, rank, local_rank) from the torchrun environment; (1, 0, 0) outside it."""
    return (int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")),
            int(os.environ.get("LOCAL_RANK", "0")))


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced slice [lo, hi) of `total` requests for `rank` (first ranks get the remainder)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(total, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def vocab_shard(vocab: int, world: int, rank: int, align: int = 128) -> Tuple[int, int]:
    """Slice of the vocabulary owned by `rank`, aligned to the GEMM's feature tile."""
    per = -(-vocab // world)
    per = -(-per // align) * align
    lo = min(rank * per, vocab)
    return lo, min(lo + per, vocab)


def _tensor(values, device):
    import torch
    return torch.tensor(np.asarray(values, dtype=np.float64), dtype=torch.float64, device=device)


def reduce_max(value: float, device: str = "cpu", group=None) -> float:
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = _tensor([value], device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def reduce_sum(value: float, device: str = "cpu", group=None) -> float:
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = _tensor([value], device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return float(t.item())


def merge_softmax_partials(maxes: np.ndarray, sums: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Merge per-shard (max, sum exp(x - max)) along axis 0 into the global pair, in float64."""
    maxes = np.asarray(maxes, dtype=np.float64)
    sums = np.asarray(sums, dtype=np.float64)
    m = maxes.max(axis=0)
    with np.errstate(invalid="ignore"):
        scale = np.where(np.isneginf(maxes), 0.0, np.exp(maxes - m))
    return m, (sums * scale).sum(axis=0)


def combine_softmax_partials(local_max: np.ndarray, local_sum: np.ndarray, device: str = "cpu",
                             group=None) -> Tuple[np.ndarray, np.ndarray]:
    """All-gather every rank's per-row (max, sum) and merge them: identical result on every rank."""
    import torch
    import torch.distributed as dist
    lm = np.asarray(local_max, dtype=np.float64)
    ls = np.asarray(local_sum, dtype=np.float64)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return merge_softmax_partials(lm[None], ls[None])
    world = dist.get_world_size(group)
    mine = torch.from_numpy(np.stack([lm, ls])).to(device)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=group)
    allp = torch.stack(gathered).cpu().numpy()
    return merge_softmax_partials(allp[:, 0], allp[:, 1])


def sharded_accept(p_shard, q_shard, draft_tokens, u_accept, u_sample, v_lo: int, temperature: float = 1.0,
                   bonus: bool = True, group=None):
    """Rejection-sampling (or greedy) acceptance over a vocabulary split across the ranks of `group`, on host arrays:
    this rank holds columns [v_lo, v_lo + Vs) of the logits of all rows.  Every rank returns the same
    (accept_len int32 [B], tokens int64 [B, k+1]) as the unsharded rule on the concatenated logits.  The protocol
    (three small all-gathers) lives in `versenext_b200.sharded`, which also drives device-resident logits."""
    import torch.distributed as dist
    from .sharded import HostShardOps, ShardedAccept, run_distributed
    rank = dist.get_rank(group) if (dist.is_available() and dist.is_initialized()) else 0
    ops = HostShardOps(p_shard, q_shard, temperature)
    return run_distributed(ShardedAccept(ops, draft_tokens, u_accept, u_sample, v_lo, rank, temperature, bonus), group)
