"""Acceptance over a vocabulary split across ranks (the exchange step of a sharded LM head).

Every rank holds columns [v_lo, v_lo + Vs) of the target and draft logits of ALL rows.  Three small exchanges make
every rank take identical decisions without moving logits:

  1. per row (max, sum exp) of the shard and the shard's logit of the draft token (-inf when another shard owns it)
     -> global softmax statistics and p(x), q(x);
  2. per sequence that samples, the shard's residual mass sum max(0, p - q) (and sum p for the fallback)
     -> which shard holds the sampled token, shards taken in ascending token order;
  3. the token picked inside that shard.

The arithmetic is the acceptance contract of the single-GPU kernels: float32 exp(x - max), float64 sums, accept iff
u * q(x) < p(x), inverse CDF over ascending token ids.  The reference has no sharded head; this file has no
counterpart there.

`ShardedAccept` runs the protocol in phases so that the same code serves a real process group
(`run_distributed`: one all-gather per phase) and a single process that walks all shards (`run_emulated`, used by the
tests).  The per-shard arithmetic comes from `HostShardOps` (NumPy) or `DeviceShardOps` (`vn_row_stats`,
`vn_row_residual`, `vn_row_pick` on device-resident logits).
"""

from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import numpy as np

F32 = np.float32


def _ptr(a):
    return None if a is None else C.c_void_p(a.ptr)


# ---------------------------------------------------------------------------------------------------------
# per-shard arithmetic
# ---------------------------------------------------------------------------------------------------------
class HostShardOps:
    """NumPy restatement of the row-level kernels; p [B, k+1, Vs], q [B, k, Vs] or None (point-mass proposals)."""

    def __init__(self, p_shard, q_shard, temperature: float):
        t = F32(max(temperature, 1e-8))
        self.p = np.asarray(p_shard, dtype=F32)
        self.q = None if q_shard is None else np.asarray(q_shard, dtype=F32)
        if temperature > 0 and temperature != 1.0:
            self.p = (self.p / t).astype(F32)
            if self.q is not None:
                self.q = (self.q / t).astype(F32)
        self.Vs = self.p.shape[-1]

    @staticmethod
    def _stats(x, tokens):
        if x.shape[-1] == 0:
            shape = x.shape[:-1]
            return np.full(shape, -np.inf), np.zeros(shape), np.full(shape, -np.inf)
        m = np.max(x, axis=-1)
        with np.errstate(invalid="ignore"):
            e = np.exp(x - m[..., None]).astype(F32)
        e = np.where(np.isneginf(m)[..., None], F32(0), e)
        s = np.sum(e, axis=-1, dtype=np.float64)
        inside = (tokens >= 0) & (tokens < x.shape[-1])
        loc = np.clip(tokens, 0, x.shape[-1] - 1)
        xt = np.take_along_axis(x, loc[..., None], axis=-1)[..., 0]
        return m.astype(np.float64), s, np.where(inside, xt, -np.inf).astype(np.float64)

    def stats(self, tokens_p, tokens_q):
        """tokens_* [B, rows] local column of the token whose logit is wanted (-1: none)."""
        out = [self._stats(self.p, tokens_p)]
        if self.q is not None:
            out.append(self._stats(self.q, tokens_q))
        return out

    def argmax(self):
        if self.Vs == 0:
            return np.full(self.p.shape[:-1], -np.inf), np.zeros(self.p.shape[:-1], np.int64)
        return self.p.max(axis=-1).astype(np.float64), self.p.argmax(axis=-1).astype(np.int64)

    def _weights(self, b, row, mode, mp, sp, mq, sq, removed):
        pr = np.exp(self.p[b, row] - F32(mp)).astype(F32).astype(np.float64) / sp
        if mode == 2:
            return pr, pr
        if mode == 3:
            r = pr.copy()
            if 0 <= removed < self.Vs:
                r[removed] = 0.0
            return r, pr
        qr = np.exp(self.q[b, row] - F32(mq)).astype(F32).astype(np.float64) / sq
        return np.maximum(pr - qr, 0.0), pr

    def residual(self, rows, mode, mp, sp, mq, sq, removed):
        B = len(rows)
        mass = np.zeros((B, 2))
        for b in range(B):
            if mode[b]:
                r, pr = self._weights(b, rows[b], mode[b], mp[b], sp[b], mq[b], sq[b], removed[b])
                mass[b] = r.sum(dtype=np.float64), pr.sum(dtype=np.float64)
        return mass

    def pick(self, rows, mode, mp, sp, mq, sq, removed, frac):
        B = len(rows)
        tok = np.full(B, -1, dtype=np.int64)
        for b in range(B):
            if not mode[b]:
                continue
            r, pr = self._weights(b, rows[b], mode[b], mp[b], sp[b], mq[b], sq[b], removed[b])
            w = r if r.sum() > 0.0 else pr
            c = np.cumsum(w, dtype=np.float64)
            t = int(np.searchsorted(c, np.float64(frac[b]) * c[-1], side="right"))
            if t >= len(c):
                nz = np.nonzero(w > 0.0)[0]
                t = int(nz[-1]) if len(nz) else len(c) - 1
            tok[b] = t
        return tok


class DeviceShardOps:
    """The same quantities from device-resident logits through the C ABI.

    p_dev: DeviceArray [B, k+1, Vs] float32, q_dev: DeviceArray [B, k, Vs] or None."""

    def __init__(self, ctx, p_dev, q_dev, temperature: float):
        self.ctx, self.p, self.q = ctx, p_dev, q_dev
        self.temperature = float(temperature) if temperature > 0 else 1.0
        self.B, self.np_, self.Vs = p_dev.shape
        self.nq = 0 if q_dev is None else q_dev.shape[1]

    def _row_stats(self, arr, rows_per_seq, tokens):
        ctx, R = self.ctx, self.B * rows_per_seq
        tok = ctx.from_numpy(np.ascontiguousarray(tokens, dtype=np.int64).reshape(R))
        m, s, x = ctx.empty((R,), np.float32), ctx.empty((R,), np.float64), ctx.empty((R,), np.float32)
        ctx._check(ctx.lib.vn_row_stats(ctx.handle, _ptr(arr), self.Vs, R, self.Vs, self.temperature, _ptr(tok),
                                        _ptr(m), _ptr(s), _ptr(x)))
        shape = (self.B, rows_per_seq)
        return (m.numpy().astype(np.float64).reshape(shape), s.numpy().reshape(shape),
                x.numpy().astype(np.float64).reshape(shape))

    def stats(self, tokens_p, tokens_q):
        out = [self._row_stats(self.p, self.np_, tokens_p)]
        if self.q is not None:
            out.append(self._row_stats(self.q, self.nq, tokens_q))
        return out

    def argmax(self):
        from . import sampling
        idx = sampling.argmax(self.ctx, self.p.reshape(self.B * self.np_, self.Vs)).numpy().reshape(self.B, self.np_)
        _, _, x = self._row_stats(self.p, self.np_, idx)       # temperature only scales by a positive constant
        return x, idx.astype(np.int64)

    def _args(self, rows, mode, mp, sp, mq, sq, removed):
        """Common arguments of vn_row_residual / vn_row_pick: the sampled row of every sequence copied into a
        compact [B, Vs] block (one row per sequence has no single pitch in the [B, rows, Vs] tensor)."""
        ctx, B = self.ctx, self.B
        rows = np.asarray(rows, dtype=np.int64)
        mode = np.asarray(mode, dtype=np.int32)
        p_rows = self._gather_rows(self.p, self.np_, rows)
        need_q = self.q is not None and bool(np.any(mode == 1))
        q_rows = self._gather_rows(self.q, self.nq, rows) if need_q else None
        d = lambda a, dt: ctx.from_numpy(np.ascontiguousarray(a, dtype=dt))
        keep = [p_rows, q_rows, d(mode, np.int32), d(mp, np.float32), d(sp, np.float64),
                d(mq, np.float32) if need_q else None, d(sq, np.float64) if need_q else None, d(removed, np.int64)]
        args = [ctx.handle, _ptr(p_rows), self.Vs, _ptr(q_rows), self.Vs if need_q else 0, B, self.Vs,
                self.temperature] + [_ptr(a) for a in keep[2:]]
        return args, keep

    def _gather_rows(self, arr, n_rows, rows):
        ctx = self.ctx
        out = ctx.empty((self.B, self.Vs), np.float32)
        flat = arr.reshape(self.B * n_rows, self.Vs)
        for b in range(self.B):
            r = int(min(max(rows[b], 0), n_rows - 1))
            ctx._check(ctx.lib.vn_d2d(ctx.handle, C.c_void_p(out.ptr + b * self.Vs * 4),
                                      C.c_void_p(flat.ptr + (b * n_rows + r) * self.Vs * 4), self.Vs * 4))
        return out

    def residual(self, rows, mode, mp, sp, mq, sq, removed):
        ctx = self.ctx
        args, keep = self._args(rows, mode, mp, sp, mq, sq, removed)
        out = ctx.empty((self.B, 2), np.float64)
        ctx._check(ctx.lib.vn_row_residual(*args, _ptr(out)))
        return out.numpy()

    def pick(self, rows, mode, mp, sp, mq, sq, removed, frac):
        ctx = self.ctx
        args, keep = self._args(rows, mode, mp, sp, mq, sq, removed)
        u = ctx.from_numpy(np.ascontiguousarray(frac, dtype=np.float32))
        out = ctx.from_numpy(np.full(self.B, -1, dtype=np.int64))
        ctx._check(ctx.lib.vn_row_pick(*args, _ptr(u), _ptr(out)))
        return out.numpy()


# ---------------------------------------------------------------------------------------------------------
# the protocol
# ---------------------------------------------------------------------------------------------------------
def _merge(maxes, sums):
    m = maxes.max(axis=0)
    with np.errstate(invalid="ignore"):
        scale = np.where(np.isneginf(maxes), 0.0, np.exp(maxes - m))
    return m, (sums * scale).sum(axis=0)


class ShardedAccept:
    """One rank's side of the protocol.  ops: HostShardOps | DeviceShardOps over this rank's columns."""

    def __init__(self, ops, draft_tokens, u_accept, u_sample, v_lo: int, rank: int, temperature: float = 1.0,
                 bonus: bool = True):
        self.ops, self.v_lo, self.rank, self.bonus = ops, int(v_lo), int(rank), bool(bonus)
        self.greedy = temperature <= 0.0
        self.draft = np.asarray(draft_tokens, dtype=np.int64)
        self.B, self.k = self.draft.shape
        self.ua = np.asarray(u_accept, dtype=np.float32) if u_accept is not None else None
        self.us = np.asarray(u_sample, dtype=np.float32) if u_sample is not None else None
        if not self.greedy and (self.ua is None or self.us is None):
            raise ValueError("the host protocol needs u_accept (B, k) and u_sample (B, k + 1) for the stochastic rule; "
                             "the device path (vn_shard_accept) draws its own Philox numbers")
        self.acc = np.zeros(self.B, dtype=np.int32)
        self.out = np.full((self.B, self.k + 1), -1, dtype=np.int64)

    # -- exchange 1 ---------------------------------------------------------------------------------
    def phase1(self) -> np.ndarray:
        B, k = self.B, self.k
        if self.greedy:
            mx, am = self.ops.argmax()
            return np.stack([mx, (am + self.v_lo).astype(np.float64)])
        local = self.draft - self.v_lo                                 # outside [0, Vs): owned by another shard
        tp = np.concatenate([local, np.full((B, 1), -1, np.int64)], axis=1)
        st = self.ops.stats(tp, local)
        pack = list(st[0])
        self.has_q = len(st) > 1
        if self.has_q:
            pad = lambda a, v: np.concatenate([a, np.full((B, 1), v)], axis=1)
            pack += [pad(st[1][0], -np.inf), pad(st[1][1], 0.0), pad(st[1][2], -np.inf)]
        return np.stack(pack)

    # -- decisions + exchange 2 -------------------------------------------------------------------
    def phase2(self, g: np.ndarray) -> np.ndarray:
        B, k = self.B, self.k
        if self.greedy:
            best = g[:, 0].max(axis=0)
            pred = np.where(g[:, 0] == best, g[:, 1], np.inf).min(axis=0).astype(np.int64)   # ties: lowest id
            for b in range(B):
                n = 0
                while n < k and self.draft[b, n] == pred[b, n]:
                    self.out[b, n] = self.draft[b, n]
                    n += 1
                self.acc[b] = n
                if n < k:
                    self.out[b, n] = pred[b, n]
                elif self.bonus:
                    self.out[b, k] = pred[b, k]
            return np.zeros((B, 2))
        self.PM, self.PS = _merge(g[:, 0], g[:, 1])
        PX = g[:, 2].max(axis=0)
        with np.errstate(invalid="ignore"):
            pp = np.where(np.isneginf(PX), 0.0, np.exp((PX - self.PM).astype(F32)).astype(np.float64) / self.PS)
            if self.has_q:
                self.QM, self.QS = _merge(g[:, 3], g[:, 4])
                QX = g[:, 5].max(axis=0)
                qq = np.where(np.isneginf(QX), 0.0, np.exp((QX - self.QM).astype(F32)).astype(np.float64) / self.QS)
            else:
                self.QM = np.zeros_like(self.PM)
                self.QS = np.ones_like(self.PS)
                qq = np.ones_like(pp)
        self.rows = np.zeros(B, dtype=np.int64)
        self.mode = np.zeros(B, dtype=np.int32)
        for b in range(B):
            n = 0
            while n < k and np.float64(self.ua[b, n]) * qq[b, n] < pp[b, n]:
                self.out[b, n] = self.draft[b, n]
                n += 1
            self.acc[b] = n
            if n < k:
                self.rows[b], self.mode[b] = n, (1 if self.has_q else 3)
            elif self.bonus:
                self.rows[b], self.mode[b] = k, 2
        idx = np.arange(B)
        self.args = (self.PM[idx, self.rows], self.PS[idx, self.rows], self.QM[idx, self.rows],
                     self.QS[idx, self.rows],
                     np.where(self.mode == 3, self.draft[idx, np.minimum(self.rows, k - 1)] - self.v_lo, -1))
        return self.ops.residual(self.rows, self.mode, *self.args)

    # -- exchange 3 ---------------------------------------------------------------------------------
    def phase3(self, gm: np.ndarray) -> np.ndarray:
        B = self.B
        picked = np.full(B, -1.0)
        if self.greedy:
            return picked
        world = gm.shape[0]
        mode = np.zeros(B, dtype=np.int32)
        frac = np.zeros(B, dtype=np.float64)
        for b in range(B):
            if not self.mode[b]:
                continue
            plain = not (gm[:, b, 0].sum() > 0.0)                       # residual vanished: sample p itself
            shard_mass = gm[:, b, 1 if plain else 0]
            cum = np.cumsum(shard_mass)
            target = np.float64(self.us[b, self.rows[b]]) * cum[-1]
            owner = int(np.searchsorted(cum, target, side="right"))
            if owner >= world:                                          # rounding: last shard that has weight
                nz = np.nonzero(shard_mass > 0.0)[0]
                owner = int(nz[-1]) if len(nz) else world - 1
                target = cum[owner]
            if owner == self.rank:
                mode[b] = 2 if plain else self.mode[b]
                before = cum[owner] - shard_mass[owner]
                frac[b] = min(max((target - before) / shard_mass[owner], 0.0), 1.0) if shard_mass[owner] > 0 else 0.0
        if mode.any():
            tok = self.ops.pick(self.rows, mode, *self.args, frac)
            picked = np.where(mode != 0, tok + self.v_lo, -1).astype(np.float64)
        return picked

    def finish(self, gp: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
        if not self.greedy:
            tok = gp.max(axis=0).astype(np.int64)
            for b in range(self.B):
                if self.mode[b]:
                    self.out[b, self.rows[b]] = tok[b]
        return self.acc, self.out


def _all_gather(arr: np.ndarray, group=None) -> np.ndarray:
    import torch
    import torch.distributed as dist
    a = np.ascontiguousarray(arr, dtype=np.float64)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return a[None]
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    mine = torch.from_numpy(a).to(dev)
    out = [torch.empty_like(mine) for _ in range(dist.get_world_size(group))]
    dist.all_gather(out, mine, group=group)
    return torch.stack(out).cpu().numpy()


def run_distributed(sa: ShardedAccept, group=None):
    """One rank of a real process group (gloo or NCCL): three all-gathers of a few numbers per row."""
    g1 = _all_gather(sa.phase1(), group)
    g2 = _all_gather(sa.phase2(g1), group)
    g3 = _all_gather(sa.phase3(g2), group)
    return sa.finish(g3)


def run_emulated(parts: Sequence[ShardedAccept]):
    """All shards in one process (tests; one GPU standing in for several): returns every shard's result."""
    g1 = np.stack([s.phase1() for s in parts])
    g2 = np.stack([s.phase2(g1) for s in parts])
    g3 = np.stack([s.phase3(g2) for s in parts])
    return [s.finish(g3) for s in parts]
