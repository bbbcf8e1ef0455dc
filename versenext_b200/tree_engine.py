"""Speculative decoding with TREE proposals (greedy rule, or stochastic with `temperature > 0`).

A round: the draft model expands a fixed tree under every request's last committed token -- the children of a node
are the draft's m most likely next tokens there, m = the node's number of children -- the target scores all nodes
in one forward (ancestor bit mask, `parents=` of `vn_model_forward`), and `vn_tree_accept_greedy` walks from the
root along the children that carry the target's own arg-max.  The committed tokens are by construction the target's
greedy continuation: the stream equals `VerseNexLM.generate(..., temperature=0)` of the target alone, whatever the
draft and the tree (what the reference's greedy rule guarantees for a chain, speculative.py:280-287).

With `temperature > 0` (and `0 < top_k < vocab`) the walk is stochastic: the children of a node are still the draft's
m best tokens, i.e. FIXED proposals, so a child is tested by rejection sampling with a point-mass proposal -- child
with token x accepted iff u * R < p(x), R the target mass not yet rejected at that node -- and where no child passes
the node's token is drawn from the target's distribution without the rejected children (`vn_tree_accept_sample`).
Every committed token then has exactly the probability the target alone (softmax(logits / T) over its top-k set)
gives it.

Everything stays on the device (tokens, arg-max, path, cache commits), so after the first, eager round the launch
sequence is replayed from a CUDA graph like the chain engine's (the draft's per-level trees are the first nodes of one
tree, whose masks a model uploads once).

`parents` describes the tree in breadth-first order: parents[i] = index of node i's parent, -1 for the first level;
depth never decreases along the list and the children of a node are consecutive.  The benchmark's 16-node tree is
`[-1, -1, -1, -1, 0, 0, 1, 1, 4, 4, 5, 5, 6, 6, 7, 7]` (4 roots, two of them expanded twice over, depth 3).
"""

from __future__ import annotations

import ctypes as C
from typing import List, Sequence

import numpy as np

from .engine import SpecEngine
from .model import _ptr


class TreeSpecEngine(SpecEngine):
    def __init__(self, target, draft, parents: Sequence[int], max_batch: int, max_seq: int,
                 max_new_tokens: int = 4096, graph: bool = True, temperature: float = 0.0, top_k: int = 0, seed: int = 0):
        parents = [int(p) for p in parents]
        n = len(parents)
        if n < 1 or n > 63:
            raise ValueError("a tree has 1 to 63 nodes")
        depth = []
        for i, p in enumerate(parents):
            if p < -1 or p >= i:
                raise ValueError(f"parents[{i}] = {p}: a parent comes before its children (-1: first level)")
            depth.append(1 if p < 0 else depth[p] + 1)
        if any(depth[i] < depth[i - 1] for i in range(1, n)):
            raise ValueError("nodes must be listed breadth first (depth never decreases)")
        kids: List[List[int]] = [[] for _ in range(n + 1)]          # kids[0]: first level, kids[i + 1]: node i
        for i, p in enumerate(parents):
            kids[p + 1].append(i)
        for ks in kids:
            if ks and ks != list(range(ks[0], ks[0] + len(ks))):
                raise ValueError("the children of a node must be consecutive")
            if len(ks) > 8:
                raise ValueError("at most 8 children per node")
        D = max(depth)
        super().__init__(target, draft, max_batch, max_seq, k=D, temperature=0.0, top_k=0, seed=int(seed), bonus=True,
                         max_new_tokens=max_new_tokens, graph=graph)
        ctx, B, V = self.ctx, self.B, self.V
        self.tree_temperature, self.tree_top_k = float(temperature), int(top_k or 0)
        if self.tree_temperature > 0 and not (0 < self.tree_top_k < V):
            raise ValueError("stochastic tree acceptance works on the top-k lists: 0 < top_k < vocab_size is needed")
        self.parents, self.depth, self.kids, self.n_nodes, self.D = parents, depth, kids, n, D
        self.T = n + 1                                   # verify rows per request: last committed token + the nodes
        self.n_verify = self.T                           # what a round appends to the target cache before the commit
        # the draft scores every node that has children; nodes of depth <= D - 1 form a prefix of the list
        self.n_inner = sum(1 for d in depth if d < D)
        self.node_tokens = ctx.zeros((B, n), np.int64)
        self.verify_tokens = ctx.zeros((B, self.T), np.int64)
        self.root_logits = ctx.empty((B, V), np.float32)
        self.d_logits = ctx.empty((B, max(self.n_inner, 1), V), np.float32)
        self.p_logits = ctx.empty((B, self.T, V), np.float32)
        self.target_arg = ctx.zeros((B, self.T), np.int64)
        self.keep_t = ctx.zeros((B, D + 1), np.int32)
        self.keep_d = ctx.zeros((B, D + 1), np.int32)
        self.parent_rows = ctx.from_numpy(np.array([-1] + [p + 1 for p in parents], np.int32))
        if self.tree_temperature > 0:     # kept top-k lists of all target rows, and the (unused) per-row draws
            self.p_lists = ctx.empty((B * self.T * self.row_bytes,), np.uint8)
            self.row_draw = ctx.zeros((B * self.T,), np.int64)
        self.q_logits = None                             # the chain engine's proposal buffers are not used
        self.step_tokens = self.draft_tokens = None
        # per level: the tokens of the nodes known so far (depth <= level), a fixed buffer so that a graph can hold it
        self.level_tokens = {lv: ctx.zeros((B, sum(1 for d in depth if d <= lv)), np.int64) for lv in range(1, D)}

    # -- one round -----------------------------------------------------------------
    def _issue_round(self, draft_part: bool = True):
        ctx, lib = self.ctx, self.ctx.lib
        ctx._check(lib.vn_set_offset_source(ctx.handle, _ptr(self.round_dev)))     # fresh Philox numbers every round
        try:
            self._issue_tree_round(draft_part)
        finally:
            ctx._check(lib.vn_set_offset_source(ctx.handle, None))

    def _issue_tree_round(self, draft_part: bool = True):
        ctx, lib, B, V, n, T, D = self.ctx, self.ctx.lib, self.B, self.V, self.n_nodes, self.T, self.D
        i64 = 8
        if draft_part:
            # first level: the draft's distribution after the last committed token (the forward consumes the last two)
            self.draft.forward_cached(self.pair, self.d_cache, last_only=True, out_logits=self.root_logits.reshape(B, 1, V),
                                      slot_offset=0)
            m0 = len(self.kids[0])
            ctx._check(lib.vn_top_m(ctx.handle, _ptr(self.root_logits), V, B, V, m0, _ptr(self.node_tokens), n))
            # deeper levels: forward the tree as far as it is known (nodes of depth <= level, behind the two tokens
            # above), read the rows of the level's nodes that have children
            for level in range(1, D):
                toks = self.level_tokens[level]
                cnt = toks.shape[1]
                ctx._check(lib.vn_copy_2d(ctx.handle, _ptr(toks), cnt * i64, _ptr(self.node_tokens), n * i64, cnt * i64, B))
                lg = self.d_logits.reshape(-1)[:B * cnt * V].reshape(B, cnt, V)
                self.draft.forward_cached(toks, self.d_cache, parents=self.parents[:cnt], out_logits=lg, slot_offset=2)
                for i in range(cnt):
                    if self.depth[i] == level and self.kids[i + 1]:
                        ks = self.kids[i + 1]
                        ctx._check(lib.vn_top_m(ctx.handle, C.c_void_p(lg.ptr + i * V * 4), cnt * V, B, V, len(ks),
                                                C.c_void_p(self.node_tokens.ptr + ks[0] * i64), n))
        # the target scores (last committed token, nodes) in one forward
        ctx._check(lib.vn_copy_2d(ctx.handle, _ptr(self.verify_tokens), T * i64, C.c_void_p(self.pair.ptr + i64), 2 * i64,
                                  i64, B))
        ctx._check(lib.vn_copy_2d(ctx.handle, C.c_void_p(self.verify_tokens.ptr + i64), T * i64, _ptr(self.node_tokens),
                                  n * i64, n * i64, B))
        self.target.forward_cached(self.verify_tokens, self.t_cache, parents=[-1] + [p + 1 for p in self.parents],
                                   out_logits=self.p_logits)
        if self.tree_temperature > 0:
            ctx._check(lib.vn_sample_lists(ctx.handle, _ptr(self.p_logits), V, B * T, V, self.tree_temperature,
                                           self.tree_top_k, None, self.seed, 0, 0, 7, _ptr(self.row_draw), _ptr(self.p_lists)))
            ctx._check(lib.vn_tree_accept_sample(ctx.handle, _ptr(self.p_lists), _ptr(self.verify_tokens),
                                                 _ptr(self.parent_rows), B, T, D, None, None, self.seed, 0,
                                                 _ptr(self.accept_len), _ptr(self.out_tokens), _ptr(self.keep_t),
                                                 _ptr(self.keep_d)))
        else:
            ctx._check(lib.vn_sample(ctx.handle, _ptr(self.p_logits), V, B * T, V, 0.0, 0, None, 0, 0, 0, 0,
                                     _ptr(self.target_arg)))
            ctx._check(lib.vn_tree_accept_greedy(ctx.handle, _ptr(self.verify_tokens), _ptr(self.target_arg),
                                                 _ptr(self.parent_rows), B, T, D, _ptr(self.accept_len),
                                                 _ptr(self.out_tokens), _ptr(self.keep_t), _ptr(self.keep_d)))
        ctx._check(lib.vn_spec_advance(ctx.handle, _ptr(self.out_tokens), B, D, _ptr(self.pair), _ptr(self.history),
                                       self.cap, _ptr(self.count), _ptr(self.n_commit)))
        # both caches keep (accepted + 1) of the entries appended this round: the accepted path, compacted in place
        ctx._check(lib.vn_kv_commit(self.t_cache.handle, T, _ptr(self.keep_t), D + 1, _ptr(self.n_commit), 0))
        if draft_part:
            ctx._check(lib.vn_kv_commit(self.d_cache.handle, 2 + self.n_inner, _ptr(self.keep_d), D + 1,
                                        _ptr(self.n_commit), 0))

    def step(self):
        before = self._len_bound
        super().step()                       # eager first, then the captured graph
        self._len_bound = before + self.D + 1   # at most depth + 1 of the appended entries stay

    def verify_accept_only(self, graph: bool = False):
        raise NotImplementedError("the tree engine has no separate verify step")
