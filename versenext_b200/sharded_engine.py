"""Speculative decoding with requests AND the LM head split over ranks (the quantised-serving configuration's data flow).

Every rank owns `B` requests (both models and both KV caches live on its GPU, as in `SpecEngine`) and the
vocabulary columns `vocab_shard(V, world, rank)` of the target and draft heads.  A round differs from
`SpecEngine`'s only between the target forward and the bookkeeping, and nothing in it touches the host:

  target forward (no logits)
  -> NCCL all-gather of the final-norm hidden rows, the draft's hidden rows and the proposals of all ranks' requests
     (three device buffers, on the library's stream)
  -> this rank's columns of every row (`vn_model_head`)
  -> `vn_shard_accept`: per-row softmax statistics, residual masses and the picked token cross the ranks in three
     more all-gathers of a few numbers per row; every rank takes the same decisions on the device
  -> this rank's own slice of the decisions goes into the device-resident round state.

The draft still samples its proposals from its own full head (it is small); only its hidden rows travel so that
every rank can form q on its columns.  Full-vocabulary rule only (top_k = 0).  Rank r draws its Philox numbers with
`seed + r * SEED_STRIDE`, so that requests on different ranks do not share uniforms and a rank's plain `SpecEngine`
built with that seed commits the same tokens.

`ShardedSpecEngine(..., comm=None)` is a world of one (no NCCL needed); `sharded.ShardedAccept` keeps the same
protocol on host arrays for process groups without GPUs (the gloo tests).
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from .dist import vocab_shard
from .engine import PURPOSE_DRAFT, SpecEngine
from .model import _ptr

SEED_STRIDE = 0x9E3779B97F4A7C15
_MASK64 = (1 << 64) - 1


def rank_seed(seed: int, rank: int) -> int:
    """The Philox seed rank `rank` draws with when the job's seed is `seed`."""
    return (int(seed) + int(rank) * SEED_STRIDE) & _MASK64


class ShardedSpecEngine(SpecEngine):
    def __init__(self, target, draft, max_batch: int, max_seq: int, k: int = 4, temperature: float = 1.0,
                 seed: int = 0, bonus: bool = True, max_new_tokens: int = 4096, comm=None, align: int = 128):
        if not bonus:
            raise ValueError("the sharded round always scores k + 1 positions")
        if temperature <= 0:
            raise ValueError("the sharded round implements the stochastic rule (temperature > 0)")
        self.comm = comm
        self.world = comm.world if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.base_seed = int(seed) & _MASK64
        super().__init__(target, draft, max_batch, max_seq, k=k, temperature=temperature, top_k=0,
                         seed=rank_seed(seed, self.rank), bonus=bonus, max_new_tokens=max_new_tokens, graph=False)
        ctx, B, V, W = self.ctx, self.B, self.V, self.world
        self.v_lo, self.v_hi = vocab_shard(V, W, self.rank, align=align)
        self.n_cols = self.v_hi - self.v_lo
        D, Dd = target.dim, draft.dim
        f32 = np.float32
        self.th_send = ctx.empty((B, k + 1, D), f32)
        self.dh_steps = ctx.empty((k, B, Dd), f32)         # step-major, as the draft produces them
        self.dh_send = ctx.empty((B, k, Dd), f32)          # request-major, as the head wants them
        self.th_all = ctx.empty((W * B * (k + 1), D), f32)
        self.dh_all = ctx.empty((W * B * k, Dd), f32)
        self.draft_all = ctx.empty((W * B, k), np.int64)
        self.p_sh = ctx.empty((W * B * (k + 1), max(self.n_cols, 1)), f32)
        self.q_sh = ctx.empty((W * B * k, max(self.n_cols, 1)), f32)
        self.len_all = ctx.zeros((W * B,), np.int32)
        self.tok_all = ctx.zeros((W * B, k + 1), np.int64)

    def _gather(self, send, recv):
        if self.comm is not None and self.world > 1:
            self.comm.all_gather(send, recv)
        else:
            self.ctx._check(self.ctx.lib.vn_d2d(self.ctx.handle, _ptr(recv), _ptr(send), send.nbytes))

    def step(self):
        self._check_capacity()
        ctx, lib, B, k, V, W = self.ctx, self.ctx.lib, self.B, self.k, self.V, self.world
        Dd = self.draft.dim
        ctx._check(lib.vn_set_offset_source(ctx.handle, _ptr(self.round_dev)))
        try:
            # ---- draft proposals (local, full draft head) and the draft's hidden rows
            for i in range(k):
                q_i = self.q_logits[i]
                if i == 0:
                    self.draft.forward_cached(self.pair, self.d_cache, last_only=True, out_logits=q_i, want_hidden=True,
                                              out_hidden=self.dh_steps[i].reshape(B, 1, Dd), slot_offset=0)
                else:
                    self.draft.forward_cached(self.step_tokens[i - 1].reshape(B, 1), self.d_cache, last_only=True,
                                              out_logits=q_i, want_hidden=True,
                                              out_hidden=self.dh_steps[i].reshape(B, 1, Dd), slot_offset=i + 1)
                ctx._check(lib.vn_sample(ctx.handle, _ptr(q_i), V, B, V, self.temperature, 0, None, self.seed, 0, i,
                                         PURPOSE_DRAFT, _ptr(self.step_tokens[i])))
                # row (b, i) of the request-major send buffer <- row b of this step
                ctx._check(lib.vn_copy_2d(ctx.handle, C.c_void_p(self.dh_send.ptr + i * Dd * 4), k * Dd * 4,
                                          _ptr(self.dh_steps[i]), Dd * 4, Dd * 4, B))
            ctx._check(lib.vn_spec_gather(ctx.handle, _ptr(self.step_tokens), _ptr(self.pair), B, k, self.n_verify,
                                          _ptr(self.draft_tokens), _ptr(self.verify_tokens)))
            # ---- target forward over (last committed, d_0 .. d_{k-1}): hidden rows only, no head
            self.target.forward_cached(self.verify_tokens, self.t_cache, want_logits=False, want_hidden=True,
                                       out_hidden=self.th_send)
            # ---- exchange 0: hidden rows and proposals of every rank's requests, device to device
            self._gather(self.th_send, self.th_all)
            self._gather(self.dh_send, self.dh_all)
            self._gather(self.draft_tokens, self.draft_all)
            # ---- this rank's columns of every row, then the three-exchange acceptance on the device
            if self.n_cols > 0:
                ctx._check(lib.vn_model_head(self.target.handle, _ptr(self.th_all), W * B * (k + 1), self.v_lo,
                                             self.n_cols, _ptr(self.p_sh), self.n_cols))
                ctx._check(lib.vn_model_head(self.draft.handle, _ptr(self.dh_all), W * B * k, self.v_lo, self.n_cols,
                                             _ptr(self.q_sh), self.n_cols))
            ctx._check(lib.vn_shard_accept(
                ctx.handle, self.comm.handle if self.comm is not None else None, _ptr(self.p_sh), _ptr(self.q_sh),
                _ptr(self.draft_all), self.v_lo, self.n_cols, self.temperature, self.base_seed, SEED_STRIDE, 0, B, W * B,
                k, 1, _ptr(self.len_all), _ptr(self.tok_all)))
            lo = self.rank * B
            ctx._check(lib.vn_d2d(ctx.handle, _ptr(self.accept_len), _ptr(self.len_all[lo:lo + B]), B * 4))
            ctx._check(lib.vn_d2d(ctx.handle, _ptr(self.out_tokens), _ptr(self.tok_all[lo:lo + B]), B * (k + 1) * 8))
            # ---- bookkeeping and cache commits, as in SpecEngine
            ctx._check(lib.vn_spec_advance(ctx.handle, _ptr(self.out_tokens), B, k, _ptr(self.pair),
                                           _ptr(self.history), self.cap, _ptr(self.count), _ptr(self.n_commit)))
            ctx._check(lib.vn_kv_commit(self.t_cache.handle, self.n_verify, None, 0, _ptr(self.n_commit), 0))
            ctx._check(lib.vn_kv_commit(self.d_cache.handle, k + 1, None, 0, _ptr(self.n_commit), 0))
        finally:
            ctx._check(lib.vn_set_offset_source(ctx.handle, None))
        self._len_bound += self.n_verify
        self.rounds_run += 1
