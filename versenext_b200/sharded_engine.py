"""Speculative decoding with requests AND the LM head split over ranks (config 5's data flow).

Every rank owns `B` requests (both models and both KV caches live on its GPU, as in `SpecEngine`) and the
vocabulary columns `vocab_shard(V, world, rank)` of the target and draft heads.  A round differs from
`SpecEngine`'s only between the target forward and the bookkeeping:

  target forward (no logits)  ->  all-gather of the final-norm hidden rows of all ranks' requests
  ->  this rank's columns of every row (`vn_model_head`)  ->  three-exchange acceptance (`sharded.ShardedAccept`)
  ->  this rank's own decisions go back into the device-resident round state.

The draft still samples its proposals from its own full head (it is small); only its hidden rows travel so that
every rank can form q on its columns.  The exchanges carry a few numbers per row and run through
`torch.distributed` (NCCL or gloo) from host staging buffers, so a round synchronises with the host several
times: this is the functional form of the sharded path, not yet a tuned one (a tuned one all-gathers the device
buffers on the library's stream and keeps the decisions on the device).  Full-vocabulary rule only (top_k = 0).
"""

from __future__ import annotations

import numpy as np

from .dist import vocab_shard
from .engine import PURPOSE_DRAFT, SpecEngine
from .model import _ptr
from . import sampling
from .sharded import DeviceShardOps, ShardedAccept, _all_gather


class ShardedSpecEngine(SpecEngine):
    def __init__(self, target, draft, max_batch: int, max_seq: int, k: int = 4, temperature: float = 1.0,
                 seed: int = 0, bonus: bool = True, max_new_tokens: int = 4096, group=None, align: int = 128):
        super().__init__(target, draft, max_batch, max_seq, k=k, temperature=temperature, top_k=0, seed=seed,
                         bonus=bonus, max_new_tokens=max_new_tokens, graph=False)
        if not bonus:
            raise ValueError("the sharded round always scores k + 1 positions")
        import torch.distributed as dist
        self.group = group
        on = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0
        self.v_lo, self.v_hi = vocab_shard(self.V, self.world, self.rank, align=align)

    def step(self):
        self._check_capacity()
        ctx, lib, B, k, V = self.ctx, self.ctx.lib, self.B, self.k, self.V
        n_cols = self.v_hi - self.v_lo
        ctx._check(lib.vn_set_offset_source(ctx.handle, _ptr(self.round_dev)))
        try:
            # ---- draft proposals (local, full draft head) and the draft's hidden rows
            d_hidden = []
            for i in range(k):
                q_i = self.q_logits[i]
                if i == 0:
                    _, h = self.draft.forward_cached(self.pair, self.d_cache, last_only=True, out_logits=q_i,
                                                     want_hidden=True, slot_offset=0)
                else:
                    _, h = self.draft.forward_cached(self.step_tokens[i - 1].reshape(B, 1), self.d_cache,
                                                     last_only=True, out_logits=q_i, want_hidden=True, slot_offset=i + 1)
                d_hidden.append(h)
                ctx._check(lib.vn_sample(ctx.handle, _ptr(q_i), V, B, V, self.temperature, 0, None, self.seed, 0, i,
                                         PURPOSE_DRAFT, _ptr(self.step_tokens[i])))
            ctx._check(lib.vn_spec_gather(ctx.handle, _ptr(self.step_tokens), _ptr(self.pair), B, k, self.n_verify,
                                          _ptr(self.draft_tokens), _ptr(self.verify_tokens)))
            # ---- target forward over (last committed, d_0 .. d_{k-1}): hidden rows only, no head
            t_hidden = self.target.forward_cached(self.verify_tokens, self.t_cache, want_logits=False, want_hidden=True)
            # ---- exchange 0: hidden rows, proposals and uniforms of every rank's requests
            th = t_hidden.numpy().reshape(B, k + 1, -1)
            dh = np.stack([h.numpy().reshape(B, -1) for h in d_hidden], axis=1)             # [B, k, Dd]
            draft = self.draft_tokens.numpy()
            rnd = self.rounds_run
            ua = sampling.philox_uniforms(ctx, self.seed, rnd, B, k, 0)
            us = sampling.philox_uniforms(ctx, self.seed, rnd, B, k + 1, 1)
            th_all = _all_gather(th, self.group).reshape(self.world * B * (k + 1), -1).astype(np.float32)
            dh_all = _all_gather(dh, self.group).reshape(self.world * B * k, -1).astype(np.float32)
            draft_all = _all_gather(draft, self.group).reshape(self.world * B, k).astype(np.int64)
            ua_all = _all_gather(ua, self.group).reshape(self.world * B, k).astype(np.float32)
            us_all = _all_gather(us, self.group).reshape(self.world * B, k + 1).astype(np.float32)
            # ---- this rank's columns of every row, then the three-exchange acceptance
            p_sh = self.target.head_columns(th_all, self.v_lo, n_cols).reshape(self.world * B, k + 1, n_cols)
            q_sh = self.draft.head_columns(dh_all, self.v_lo, n_cols).reshape(self.world * B, k, n_cols)
            sa = ShardedAccept(DeviceShardOps(ctx, p_sh, q_sh, self.temperature), draft_all, ua_all, us_all, self.v_lo,
                               self.rank, self.temperature, True)
            g1 = _all_gather(sa.phase1(), self.group)
            g2 = _all_gather(sa.phase2(g1), self.group)
            g3 = _all_gather(sa.phase3(g2), self.group)
            acc, out = sa.finish(g3)
            mine = slice(self.rank * B, (self.rank + 1) * B)
            self.accept_len.copy_from_host(acc[mine].astype(np.int32))
            self.out_tokens.copy_from_host(out[mine].astype(np.int64))
            # ---- bookkeeping and cache commits, as in SpecEngine
            ctx._check(lib.vn_spec_advance(ctx.handle, _ptr(self.out_tokens), B, k, _ptr(self.pair),
                                           _ptr(self.history), self.cap, _ptr(self.count), _ptr(self.n_commit)))
            ctx._check(lib.vn_kv_commit(self.t_cache.handle, self.n_verify, None, 0, _ptr(self.n_commit), 0))
            ctx._check(lib.vn_kv_commit(self.d_cache.handle, k + 1, None, 0, _ptr(self.n_commit), 0))
        finally:
            ctx._check(lib.vn_set_offset_source(ctx.handle, None))
        self._len_bound += self.n_verify
        self.rounds_run += 1
