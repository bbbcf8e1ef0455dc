"""Batched speculative decoding with a draft MODEL: draft -> verify -> accept -> commit.

The reference composes this loop on the host from `VerseNexLM.forward` and
`SpeculativeDecoder.verify_then_commit` (verse_nex/speculative.py:230-310),
re-running the whole context every round and serving batch row 0 only.
Here both models keep KV caches on the device, every request of the batch
advances each round, and a round issues no host synchronisation: proposals,
acceptance results, the last committed tokens, the cache lengths and the
round counter that offsets the Philox streams all stay in device memory
(`vn_spec_gather`, `vn_accept`, `vn_spec_advance`, `vn_kv_commit`).  Because
the launch sequence of a round is then fixed, it is captured once into a CUDA
graph and replayed (`graph=True`).

Cache protocol.  With s the committed tokens of a request, at the start of a
round the target cache holds s[:-1] and the draft cache s[:-2].  The draft
first consumes (s[-2], s[-1]) in one forward, then its own proposals one at a
time; the target scores (s[-1], d_0 .. d_{k-1}) in one forward.  If n tokens
are committed, both caches keep the first n entries they appended this round
and drop the rest.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from .model import VerseNexLM, _ptr

PURPOSE_DRAFT = 2  # Philox purpose of the draft model's own sampling (0 / 1: accept test / resample)


class SpecEngine:
    def __init__(self, target: VerseNexLM, draft: VerseNexLM, max_batch: int, max_seq: int, k: int = 4,
                 temperature: float = 0.0, top_k: int = 0, seed: int = 0, bonus: bool = True,
                 max_new_tokens: int = 4096, graph: bool = True):
        if target.vocab_size != draft.vocab_size:
            raise ValueError("target and draft must share the vocabulary")
        if target.ctx is not draft.ctx:
            raise ValueError("target and draft must live on the same device")
        if k < 1 or k > 16:
            raise ValueError("k must be in [1, 16]")
        self.target, self.draft, self.ctx = target, draft, target.ctx
        self.B, self.k, self.V = int(max_batch), int(k), target.vocab_size
        self.temperature, self.top_k, self.seed, self.bonus = float(temperature), int(top_k or 0), int(seed), bool(bonus)
        self.n_verify = self.k + 1 if self.bonus else self.k
        self.max_seq = int(max_seq)
        self.t_cache = target.new_cache(self.B, max_seq)
        self.d_cache = draft.new_cache(self.B, max_seq)
        ctx, B, k, V = self.ctx, self.B, self.k, self.V
        self.cap = int(max_new_tokens) + k + 1
        self.pair = ctx.zeros((B, 2), np.int64)
        self.step_tokens = ctx.zeros((k, B), np.int64)
        self.draft_tokens = ctx.zeros((B, k), np.int64)
        self.verify_tokens = ctx.zeros((B, self.n_verify), np.int64)
        self.q_logits = ctx.empty((k, B, V), np.float32)          # step-major: row (b, i) at (i*B + b) * V
        self.p_logits = ctx.empty((B, self.n_verify, V), np.float32)
        self.accept_len = ctx.zeros((B,), np.int32)
        self.out_tokens = ctx.zeros((B, k + 1), np.int64)
        self.history = ctx.zeros((B, self.cap), np.int64)
        self.count = ctx.zeros((B,), np.int32)
        self.n_commit = ctx.zeros((B,), np.int32)
        # kept lists of the draft's top-k selection, one record per (step, request): sampled from at draft time and
        # read again as q by the acceptance step, so the draft rows are selected once per round
        self.fused_head = self.temperature > 0 and 0 < self.top_k < V
        self.row_bytes = int(ctx.lib.vn_topk_row_bytes())
        self.q_lists = ctx.empty((k * B * self.row_bytes,), np.uint8) if self.fused_head else None
        self.round_dev = ctx.zeros((1,), np.uint32)               # rounds completed; offsets the Philox streams
        self.rounds_run = 0
        self.use_graph = bool(graph)
        self._graph = None
        self._graph_verify = None
        self._eager_rounds = 0
        self._len_bound = 0        # host upper bound of the longest target-cache length

    # -- prefill -------------------------------------------------------------------
    def prefill(self, prompts):
        """prompts (B, T) int64 with T >= 2.  Fills both caches and the (s[-2], s[-1]) pair."""
        prompts = np.ascontiguousarray(prompts, dtype=np.int64)
        B, T = prompts.shape
        if B != self.B:
            raise ValueError(f"engine was built for batch {self.B}, got {B}")
        if T < 2:
            raise ValueError("prompts need at least two tokens")
        self.t_cache.reset()
        self.d_cache.reset()
        # chunk the prompt so that activation buffers stay bounded for long prompts
        chunk = max(1, 8192 // B)
        for cache, model, upto in ((self.t_cache, self.target, T - 1), (self.d_cache, self.draft, T - 2)):
            done = 0
            while done < upto:
                n = min(chunk, upto - done)
                part = self.ctx.from_numpy(prompts[:, done:done + n])
                model.forward_cached(part, cache, want_logits=False, want_hidden=True, last_only=True)
                cache.commit(n, np.full(B, n, np.int32))
                done += n
        self._prompt_len = T
        self._prompt_pair = prompts[:, -2:].copy()
        self.rewind()

    def rewind(self):
        """Back to the state right after `prefill`: generated tokens are dropped, the prompt's K/V stay in both
        caches (a sequence's entries behind its length are simply overwritten by the next rounds)."""
        T = self._prompt_len
        self.t_cache.set_lengths(np.full(self.B, T - 1, np.int32))
        self.d_cache.set_lengths(np.full(self.B, T - 2, np.int32))
        self.pair.copy_from_host(self._prompt_pair)
        for buf in (self.count, self.round_dev):
            self.ctx._check(self.ctx.lib.vn_memset(self.ctx.handle, _ptr(buf), 0, buf.nbytes))
        self.rounds_run = 0
        self._len_bound = T - 1

    # -- one round -----------------------------------------------------------------
    def _issue_round(self, draft_part: bool = True):
        """Enqueue the kernels of one round on the context's stream (no synchronisation, no allocation)."""
        ctx, lib, B, k, V = self.ctx, self.ctx.lib, self.B, self.k, self.V
        greedy = self.temperature <= 0
        ctx._check(lib.vn_set_offset_source(ctx.handle, _ptr(self.round_dev)))
        try:
            if draft_part:
                # draft: k proposals, token by token on the device; the first forward consumes the last two
                # committed tokens.  Step i's kept top-k list stays at record i * B + b for the fused verify.
                if not self.draft._finalized:
                    self.draft.finalize()
                ctx._check(lib.vn_draft_propose(
                    self.draft.handle, self.d_cache.handle, _ptr(self.pair), B, k, self.temperature, self.top_k,
                    self.seed, 0, _ptr(self.q_logits), _ptr(self.step_tokens),
                    _ptr(self.q_lists) if self.fused_head else None))
                ctx._check(lib.vn_spec_gather(ctx.handle, _ptr(self.step_tokens), _ptr(self.pair), B, k,
                                              self.n_verify, _ptr(self.draft_tokens), _ptr(self.verify_tokens)))
            # target: one forward over (last committed, d_0 .. d_{n_verify-2}), LM head and acceptance in one call;
            # with top-k sampling the head is fused with the selection and q comes from the lists kept above
            # (record of (request b, step i) at i * B + b)
            if not self.target._finalized:
                self.target.finalize()
            ctx._check(lib.vn_verify_accept(
                self.target.handle, self.t_cache.handle, _ptr(self.verify_tokens), B, self.n_verify, k,
                _ptr(self.q_lists) if self.fused_head else None, 1, B,
                None if greedy else _ptr(self.q_logits), V, B * V,
                _ptr(self.draft_tokens), None, None, self.seed, 0, self.temperature, self.top_k,
                int(self.bonus), _ptr(self.p_logits), _ptr(self.accept_len), _ptr(self.out_tokens)))
            ctx._check(lib.vn_spec_advance(ctx.handle, _ptr(self.out_tokens), B, k, _ptr(self.pair),
                                           _ptr(self.history), self.cap, _ptr(self.count), _ptr(self.n_commit)))
            # both caches keep the first n_commit entries appended this round
            ctx._check(lib.vn_kv_commit(self.t_cache.handle, self.n_verify, None, 0, _ptr(self.n_commit), 0))
            if draft_part:
                ctx._check(lib.vn_kv_commit(self.d_cache.handle, k + 1, None, 0, _ptr(self.n_commit), 0))
        finally:
            ctx._check(lib.vn_set_offset_source(ctx.handle, None))

    def _check_capacity(self):
        # the device kernels trust the cache capacity; every round appends at most n_verify entries
        if self._len_bound + self.n_verify + 1 > self.max_seq:
            lens = self.t_cache.per_seq_lens
            self._len_bound = int(lens.max())
            if self._len_bound + self.n_verify + 1 > self.max_seq:
                raise RuntimeError(f"KV cache overflow: a sequence holds {self._len_bound} of {self.max_seq} positions")

    def step(self):
        """One speculative round for the whole batch."""
        self._check_capacity()
        ctx, lib = self.ctx, self.ctx.lib
        if self.use_graph and self._eager_rounds >= 1:
            if self._graph is None:
                ctx._check(lib.vn_graph_begin(ctx.handle))
                try:
                    self._issue_round()
                finally:
                    g = C.c_void_p()
                    ctx._check(lib.vn_graph_end(ctx.handle, C.byref(g)))
                self._graph = g
            ctx._check(lib.vn_graph_launch(ctx.handle, self._graph))
        else:
            self._issue_round()          # the first round runs eagerly: buffers grow, attributes get set
            self._eager_rounds += 1
        self._len_bound += self.n_verify
        self.rounds_run += 1

    def verify_accept_only(self, graph: bool = False):
        """The verify + sample half of a round on the current proposals (for timing): target forward,
        acceptance, bookkeeping and the target cache commit; the draft cache is left alone."""
        self._check_capacity()
        ctx, lib = self.ctx, self.ctx.lib
        if graph:
            if self._graph_verify is None:
                ctx._check(lib.vn_graph_begin(ctx.handle))
                try:
                    self._issue_round(draft_part=False)
                finally:
                    g = C.c_void_p()
                    ctx._check(lib.vn_graph_end(ctx.handle, C.byref(g)))
                self._graph_verify = g
            ctx._check(lib.vn_graph_launch(ctx.handle, self._graph_verify))
        else:
            self._issue_round(draft_part=False)
        self._len_bound += self.n_verify

    # -- results --------------------------------------------------------------------
    def counts(self) -> np.ndarray:
        return self.count.numpy()

    def tokens(self, n_new: Optional[int] = None) -> np.ndarray:
        """Generated tokens per request, (B, n_new) (requests must have produced at least n_new)."""
        c = self.counts()
        n = int(c.min()) if n_new is None else int(n_new)
        if n > c.min():
            raise ValueError(f"only {int(c.min())} tokens available")
        return self.history.numpy()[:, :n]

    def generate(self, prompts, max_new_tokens: int, eos_id: Optional[int] = None):
        """Run rounds until every request has `max_new_tokens` tokens, or -- with `eos_id` -- until there is a step
        at which every request emitted EOS (the stop rule of the reference's loops, cometspark.py:862-865; rows are
        returned uncut, the caller trims at that step).  Returns (tokens (B, T + new), stats)."""
        prompts = np.ascontiguousarray(prompts, dtype=np.int64)
        if max_new_tokens + self.k + 1 > self.cap:
            raise ValueError("max_new_tokens exceeds the engine's history capacity")
        self.prefill(prompts)
        n = max_new_tokens
        while True:
            # a request gains at least one token per round: poll the counters only now and then
            c = self.counts()
            have = min(int(c.min()), max_new_tokens)
            if eos_id is not None and have > 0:
                stop = np.flatnonzero(np.all(self.history.numpy()[:, :have] == eos_id, axis=0))
                if stop.size:
                    n = int(stop[0]) + 1
                    break
            need = max_new_tokens - have
            if need <= 0:
                break
            for _ in range(max(1, need // (self.k + 1))):
                self.step()
        self.target.check()          # token ids in range, no kernel wait ran out
        self.draft.check()
        new = self.tokens(n)
        stats = dict(rounds=self.rounds_run, proposed=self.rounds_run * self.k * self.B,
                     committed=int(self.counts().sum()))
        return np.concatenate([prompts, new], axis=1), stats

    # -- serving: requests come and go, slots are reused ------------------------------------------------------
    def admit(self, slot: int, prompt):
        """Start a new request in slot `slot` (whatever ran there is dropped): its prompt is prefilled into that
        slot's rows of both caches through cache views while the other slots keep their state."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int64).reshape(-1)
        T = prompt.shape[0]
        if T < 2:
            raise ValueError("a request needs at least two prompt tokens")
        if not 0 <= slot < self.B:
            raise IndexError(f"slot {slot} outside [0, {self.B})")
        if T + self.k + 2 > self.max_seq:
            raise RuntimeError(f"prompt of {T} tokens does not fit the cache's {self.max_seq} positions")
        for cache, model, upto in ((self.t_cache, self.target, T - 1), (self.d_cache, self.draft, T - 2)):
            view = cache.view(slot, 1)
            view.reset()
            done = 0
            while done < upto:
                n = min(4096, upto - done)
                part = self.ctx.from_numpy(prompt[None, done:done + n])
                model.forward_cached(part, view, want_logits=False, want_hidden=True, last_only=True)
                view.commit(n, np.full(1, n, np.int32))
                done += n
        self.pair[slot:slot + 1].copy_from_host(prompt[None, -2:])
        cnt = self.count[slot:slot + 1]
        self.ctx._check(self.ctx.lib.vn_memset(self.ctx.handle, _ptr(cnt), 0, cnt.nbytes))
        self._len_bound = max(self._len_bound, T - 1)

    def _park(self, slot: int):
        """An idle slot keeps running (the batch shape is fixed) on an empty context, so that it cannot overflow."""
        self.t_cache.view(slot, 1).reset()
        self.d_cache.view(slot, 1).reset()
        self.pair[slot:slot + 1].copy_from_host(np.zeros((1, 2), np.int64))
        cnt = self.count[slot:slot + 1]
        self.ctx._check(self.ctx.lib.vn_memset(self.ctx.handle, _ptr(cnt), 0, cnt.nbytes))

    def serve(self, prompts, max_new_tokens, eos_id: Optional[int] = None, poll_every: int = 4):
        """Continuous batching: `prompts` is any number of requests (1-D token arrays of any lengths); at most
        `max_batch` run at a time, and a request that has produced `max_new_tokens` tokens (an int, or one per
        request) or an EOS leaves its slot to the next waiting one.  Every `poll_every` rounds the host reads the
        per-slot counters and tokens (a few KB) to find finished requests; nothing else synchronises.
        Returns the list of generated token arrays (prompt excluded, EOS included), in request order."""
        from collections import deque
        reqs = [np.ascontiguousarray(p, dtype=np.int64).reshape(-1) for p in prompts]
        limits = [int(max_new_tokens)] * len(reqs) if np.isscalar(max_new_tokens) else [int(x) for x in max_new_tokens]
        if len(limits) != len(reqs):
            raise ValueError("one max_new_tokens per request")
        if max(limits, default=0) + self.k + 1 > self.cap:
            raise ValueError("max_new_tokens exceeds the engine's history capacity")
        results = [None] * len(reqs)
        waiting = deque(range(len(reqs)))
        running = [-1] * self.B
        self.t_cache.reset()
        self.d_cache.reset()
        self._len_bound = 0
        for buf in (self.count, self.round_dev):
            self.ctx._check(self.ctx.lib.vn_memset(self.ctx.handle, _ptr(buf), 0, buf.nbytes))
        for slot in range(self.B):
            if waiting:
                running[slot] = waiting.popleft()
                self.admit(slot, reqs[running[slot]])
            else:
                self._park(slot)
        while any(r >= 0 for r in running):
            for _ in range(max(1, int(poll_every))):
                self.step()
            c = self.counts()
            h = self.history.numpy()
            for slot, r in enumerate(running):
                if r < 0:
                    self._park(slot)             # keep idle slots short
                    continue
                got = h[slot, :min(int(c[slot]), self.cap)]
                end = -1
                if eos_id is not None:
                    hit = np.flatnonzero(got[:limits[r]] == eos_id)
                    if hit.size:
                        end = int(hit[0]) + 1
                if end < 0 and got.shape[0] >= limits[r]:
                    end = limits[r]
                if end >= 0:
                    results[r] = got[:end].copy()
                    if waiting:
                        running[slot] = waiting.popleft()
                        self.admit(slot, reqs[running[slot]])
                    else:
                        running[slot] = -1
                        self._park(slot)
            if all(r < 0 for r in running):
                break
            lens = self.t_cache.per_seq_lens
            self._len_bound = int(lens.max())
        self.target.check()
        self.draft.check()
        return results

    def __del__(self):
        try:
            for name in ("_graph", "_graph_verify"):
                g = getattr(self, name, None)
                if g is not None:
                    self.ctx.lib.vn_graph_destroy(self.ctx.handle, g)
                    setattr(self, name, None)
        except Exception:
            pass
