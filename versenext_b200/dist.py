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


# ---------------------------------------------------------------------------------------------------------
# Vocabulary-sharded acceptance: the exchange protocol of a sharded LM head, on host arrays.
#
# Every rank holds columns [v_lo, v_hi) of the target and draft logits of ALL rows (the hidden states were
# all-gathered before the head).  Three small exchanges make every rank take identical decisions:
#   1. per row (max, sum exp) of the shard, and the shard's logit of the draft token (or -inf): softmax
#      statistics and p(x), q(x) without moving any logits;
#   2. per rejected (or bonus) row the shard's residual mass sum max(0, p - q): picks the shard that holds the
#      sampled token, shards taken in ascending token order;
#   3. the token picked inside that shard.
# The arithmetic follows the acceptance contract of the single-GPU kernels: float32 exp(x - max), float64 sums,
# accept iff u * q(x) < p(x), inverse CDF over ascending token ids.  The device kernels that would produce the
# per-shard partials are not built; this is the protocol they plug into, and what the CPU tests pin.
# ---------------------------------------------------------------------------------------------------------

def _all_gather_f64(arr: np.ndarray, group=None) -> np.ndarray:
    """Stack of every rank's float64 array (same shape on all ranks), rank-major."""
    import torch
    import torch.distributed as dist
    a = np.ascontiguousarray(arr, dtype=np.float64)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return a[None]
    mine = torch.from_numpy(a)
    out = [torch.empty_like(mine) for _ in range(dist.get_world_size(group))]
    dist.all_gather(out, mine, group=group)
    return torch.stack(out).numpy()


def _shard_stats(x: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """(max, sum exp(x - max)) over the last axis: float32 exp, float64 sum (empty shard: -inf, 0)."""
    if x.shape[-1] == 0:
        return np.full(x.shape[:-1], -np.inf), np.zeros(x.shape[:-1])
    m = np.max(x, axis=-1)
    with np.errstate(invalid="ignore"):
        e = np.exp(x - m[..., None]).astype(np.float32)
    e = np.where(np.isneginf(m)[..., None], np.float32(0), e)
    return m.astype(np.float64), np.sum(e, axis=-1, dtype=np.float64)


def sharded_accept(p_shard, q_shard, draft_tokens, u_accept, u_sample, v_lo: int, temperature: float = 1.0,
                   bonus: bool = True, group=None):
    """Rejection-sampling acceptance over a vocabulary split across ranks.

    p_shard [B, k+1, Vs] / q_shard [B, k, Vs]: this rank's columns [v_lo, v_lo + Vs) of the target / draft
    logits; draft_tokens [B, k] global ids; u_accept [B, k], u_sample [B, k+1].  Every rank returns the same
    (accept_len int32 [B], tokens int64 [B, k+1] padded with -1), equal to the unsharded rule on the
    concatenated logits.  temperature <= 0 selects the greedy rule (arg-max compare)."""
    p = np.asarray(p_shard, dtype=np.float32)
    draft = np.asarray(draft_tokens, dtype=np.int64)
    B, k = draft.shape
    Vs = p.shape[-1]
    greedy = temperature <= 0.0
    if not greedy and temperature != 1.0:
        p = (p / np.float32(max(temperature, 1e-8))).astype(np.float32)
    q = None
    if q_shard is not None and not greedy:
        q = np.asarray(q_shard, dtype=np.float32)
        if temperature != 1.0:
            q = (q / np.float32(max(temperature, 1e-8))).astype(np.float32)
    acc = np.zeros(B, dtype=np.int32)
    out = np.full((B, k + 1), -1, dtype=np.int64)

    if greedy:
        # exchange 1 (greedy form): the shard's maximum and where it sits; ties go to the lowest token id
        lm = p.max(axis=-1) if Vs else np.full((B, k + 1), -np.inf, np.float32)
        la = (p.argmax(axis=-1) + v_lo) if Vs else np.zeros((B, k + 1), np.int64)
        g = _all_gather_f64(np.stack([lm.astype(np.float64), la.astype(np.float64)]), group)   # [W, 2, B, k+1]
        best = g[:, 0].max(axis=0)
        cand = np.where(g[:, 0] == best, g[:, 1], np.inf)
        pred = cand.min(axis=0).astype(np.int64)
        for b in range(B):
            n = 0
            while n < k and draft[b, n] == pred[b, n]:
                out[b, n] = draft[b, n]
                n += 1
            acc[b] = n
            if n < k:
                out[b, n] = pred[b, n]
            elif bonus:
                out[b, k] = pred[b, k]
        return acc, out

    # ---- exchange 1: softmax statistics of every row and the draft tokens' logits
    pm, ps = _shard_stats(p)                                        # [B, k+1]
    in_shard = (draft >= v_lo) & (draft < v_lo + Vs)
    loc = np.clip(draft - v_lo, 0, max(Vs - 1, 0))
    rows = np.arange(B)[:, None], np.arange(k)[None, :]
    px = np.where(in_shard, p[rows[0], rows[1], loc] if Vs else -np.inf, -np.inf).astype(np.float64)
    pack = [pm, ps, np.pad(px, ((0, 0), (0, 1)), constant_values=-np.inf)]
    if q is not None:
        qm, qs = _shard_stats(q)
        qx = np.where(in_shard, q[rows[0], rows[1], loc] if Vs else -np.inf, -np.inf).astype(np.float64)
        pack += [np.pad(qm, ((0, 0), (0, 1)), constant_values=-np.inf), np.pad(qs, ((0, 0), (0, 1))),
                 np.pad(qx, ((0, 0), (0, 1)), constant_values=-np.inf)]
    g = _all_gather_f64(np.stack(pack), group)                      # [W, 3 or 6, B, k+1]
    PM, PS = merge_softmax_partials(g[:, 0], g[:, 1])
    PX = g[:, 2].max(axis=0)
    _err = np.seterr(invalid="ignore")                              # -inf - (-inf) for tokens outside the vocabulary
    prob_p = np.where(np.isneginf(PX), 0.0, np.exp((PX - PM).astype(np.float32)).astype(np.float64) / PS)
    if q is not None:
        QM, QS = merge_softmax_partials(g[:, 3], g[:, 4])
        QX = g[:, 5].max(axis=0)
        prob_q = np.where(np.isneginf(QX), 0.0, np.exp((QX - QM).astype(np.float32)).astype(np.float64) / QS)
    else:
        prob_q = np.ones((B, k + 1))                                # deterministic proposals: q(x) = 1
    np.seterr(**_err)

    # ---- decisions (identical on every rank)
    sample_row = np.full(B, -1, dtype=np.int64)                     # p row to sample from, -1: nothing to sample
    rejected = np.zeros(B, dtype=bool)
    for b in range(B):
        n = 0
        while n < k and np.float64(u_accept[b, n]) * prob_q[b, n] < prob_p[b, n]:
            out[b, n] = draft[b, n]
            n += 1
        acc[b] = n
        if n < k:
            sample_row[b], rejected[b] = n, True
        elif bonus:
            sample_row[b] = k

    # ---- exchange 2: residual mass of the shard for every row that samples
    def weights(b):
        j = int(sample_row[b])
        pr = np.exp(p[b, j] - np.float32(PM[b, j])).astype(np.float32).astype(np.float64) / PS[b, j]
        if not rejected[b]:
            return pr, pr
        if q is not None:
            qr = np.exp(q[b, j] - np.float32(QM[b, j])).astype(np.float32).astype(np.float64) / QS[b, j]
            return np.maximum(pr - qr, 0.0), pr
        r = pr.copy()
        x = int(draft[b, j]) - v_lo
        if 0 <= x < Vs:
            r[x] = 0.0                                              # q is a point mass on the rejected token
        return r, pr

    mass = np.zeros((2, B))
    wcache = {}
    for b in range(B):
        if sample_row[b] >= 0:
            r, pr = weights(b)
            wcache[b] = (r, pr)
            mass[0, b], mass[1, b] = r.sum(dtype=np.float64), pr.sum(dtype=np.float64)
    gm = _all_gather_f64(mass, group)                               # [W, 2, B]

    # ---- exchange 3: the owner of the sampled token reports it
    picked = np.full(B, -1.0)
    world = gm.shape[0]
    import torch.distributed as dist
    my_rank = dist.get_rank(group) if (dist.is_available() and dist.is_initialized()) else 0
    for b in range(B):
        if sample_row[b] < 0:
            continue
        plain = not (gm[:, 0, b].sum() > 0.0)                        # residual vanished: fall back to p itself
        col = 1 if plain else 0
        shard_mass = gm[:, col, b]
        total = shard_mass.sum()
        target = np.float64(u_sample[b, sample_row[b]]) * total
        cum = np.cumsum(shard_mass)
        owner = int(np.searchsorted(cum, target, side="right"))
        if owner >= world:                                           # rounding: last shard that has weight
            nz = np.nonzero(shard_mass > 0.0)[0]
            owner = int(nz[-1]) if len(nz) else world - 1
            target = cum[owner]                                      # past the end of that shard: its last token
        if owner == my_rank:
            w = wcache[b][col]
            before = cum[owner] - shard_mass[owner]
            c = np.cumsum(w, dtype=np.float64) + before
            t = int(np.searchsorted(c, target, side="right"))
            if t >= len(c):
                nz = np.nonzero(w > 0.0)[0]
                t = int(nz[-1]) if len(nz) else len(c) - 1
            picked[b] = t + v_lo
    gp = _all_gather_f64(picked, group)                              # [W, B]
    tok = gp.max(axis=0).astype(np.int64)
    for b in range(B):
        if sample_row[b] >= 0:
            out[b, sample_row[b]] = tok[b]
    return acc, out
