"""Stochastic acceptance on a verified tree with fixed proposals (`vn_tree_accept_sample`, `TreeSpecEngine` with
temperature > 0): decisions against the CPU oracle on injected and on Philox uniforms, the distribution of the
committed token against the target's own, and the engine's rounds (graph replay = eager, tokens inside the target's
top-k set)."""

import ctypes as C

import numpy as np
import pytest

from oracle import accept as OA
from oracle import model as OM

pytestmark = pytest.mark.gpu

CFG3_TREE = [-1, -1, -1, -1, 0, 0, 1, 1, 4, 4, 5, 5, 6, 6, 7, 7]


def _ptr(a):
    return C.c_void_p(a.ptr) if a is not None else C.c_void_p(None)


def _device_walk(ctx, logits, tokens, parent_rows, depth, temperature, top_k, u_child=None, u_sample=None, seed=0,
                 offset=0):
    """Kept lists of all rows (vn_sample_lists), then vn_tree_accept_sample."""
    lib = ctx.lib
    B, T, V = logits.shape
    lg = ctx.from_numpy(np.ascontiguousarray(logits, np.float32))
    lists = ctx.empty((B * T * int(lib.vn_topk_row_bytes()),), np.uint8)
    draws = ctx.zeros((B * T,), np.int64)
    ctx._check(lib.vn_sample_lists(ctx.handle, _ptr(lg), V, B * T, V, temperature, top_k, None, seed, 0, 0, 7,
                                   _ptr(draws), _ptr(lists)))
    tok = ctx.from_numpy(np.ascontiguousarray(tokens, np.int64))
    par = ctx.from_numpy(np.asarray(parent_rows, np.int32))
    uc = ctx.from_numpy(np.ascontiguousarray(u_child, np.float32)) if u_child is not None else None
    us = ctx.from_numpy(np.ascontiguousarray(u_sample, np.float32)) if u_sample is not None else None
    n = ctx.zeros((B,), np.int32)
    out = ctx.zeros((B, depth + 1), np.int64)
    kt = ctx.zeros((B, depth + 1), np.int32)
    kd = ctx.zeros((B, depth + 1), np.int32)
    ctx._check(lib.vn_tree_accept_sample(ctx.handle, _ptr(lists), _ptr(tok), _ptr(par), B, T, depth, _ptr(uc), _ptr(us),
                                         seed, offset, _ptr(n), _ptr(out), _ptr(kt), _ptr(kd)))
    return n.numpy(), out.numpy(), kt.numpy(), kd.numpy()


def _tree_case(rng, B, V, temperature, top_k, parents):
    """Random target logits for every row; a node's token is one of its parent's more likely tokens (so that children
    are accepted often), the first child sometimes a token outside the parent's top-k set (probability zero)."""
    T = len(parents) + 1
    parent_rows = [-1] + [p + 1 for p in parents]
    depth = max(_depths(parents))
    logits = rng.normal(0.0, 2.0, (B, T, V)).astype(np.float32)
    tokens = np.zeros((B, T), np.int64)
    tokens[:, 0] = rng.integers(0, V, B)
    for b in range(B):
        used = {}
        for r in range(1, T):
            pr = parent_rows[r]
            p = OA.softmax64(logits[b, pr], temperature, top_k)
            order = np.argsort(-p, kind="stable")
            j = used.get(pr, 0)
            used[pr] = j + 1
            tokens[b, r] = order[(j * 2 + b) % max(top_k + 2, 1)]      # distinct among the siblings; may leave the top-k set
    return logits, tokens, parent_rows, depth


def _depths(parents):
    d = []
    for p in parents:
        d.append(1 if p < 0 else d[p] + 1)
    return d


@pytest.mark.parametrize("V,top_k,temperature", [(300, 20, 0.8), (4096, 50, 1.0), (97, 5, 1.3)])
def test_tree_walk_equals_the_oracle_on_injected_and_philox_uniforms(V, top_k, temperature):
    import versenext_b200 as vn
    ctx = vn.Context.get(0)
    rng = np.random.default_rng(V)
    B = 24
    logits, tokens, parent_rows, depth = _tree_case(rng, B, V, temperature, top_k, CFG3_TREE)
    T = tokens.shape[1]
    u1 = rng.random((B, T)).astype(np.float32)
    u2 = rng.random((B, T)).astype(np.float32)
    u1[:4] = 0.0                                   # always accept where the child has any probability
    u1[4:8] = np.float32(1.0 - 2.0 ** -24)         # (almost) never accept
    want_n, want_out, want_path = OA.tree_accept_stochastic(logits, tokens, parent_rows, depth, u1, u2, temperature, top_k)
    n, out, kt, kd = _device_walk(ctx, logits, tokens, parent_rows, depth, temperature, top_k, u1, u2)
    np.testing.assert_array_equal(n, want_n)
    np.testing.assert_array_equal(out, want_out)
    np.testing.assert_array_equal(kt, want_path)
    assert n.max() == depth and n.min() == 0
    for b in range(B):                             # the draft's cache keeps slots 0, 1 and path row + 1 (one level less)
        assert list(kd[b, :2]) == [0, 1] and all(kd[b, a + 1] == kt[b, a] + 1 for a in range(1, min(n[b], depth - 1) + 1))
    # Philox: the same uniforms as vn_philox_uniform hands out (row b, position = row index, purpose 0 / 1)
    seed, offset = 77, 5
    uc = ctx.empty((B, T), np.float32)
    us = ctx.empty((B, T), np.float32)
    ctx._check(ctx.lib.vn_philox_uniform(ctx.handle, seed, offset, B, T, 0, _ptr(uc)))
    ctx._check(ctx.lib.vn_philox_uniform(ctx.handle, seed, offset, B, T, 1, _ptr(us)))
    want_n, want_out, want_path = OA.tree_accept_stochastic(logits, tokens, parent_rows, depth, uc.numpy(), us.numpy(),
                                                            temperature, top_k)
    n, out, kt, _ = _device_walk(ctx, logits, tokens, parent_rows, depth, temperature, top_k, seed=seed, offset=offset)
    np.testing.assert_array_equal(n, want_n)
    np.testing.assert_array_equal(out, want_out)
    np.testing.assert_array_equal(kt, want_path)


def test_first_committed_token_follows_the_target_distribution():
    """One row of target logits, 8192 independent requests (Philox row index), three fixed children of very different
    probability: the histogram of the first committed token is the target's top-k softmax, whatever the children."""
    import versenext_b200 as vn
    ctx = vn.Context.get(0)
    rng = np.random.default_rng(1)
    B, V, top_k, temperature = 8192, 64, 10, 0.9
    row = rng.normal(0.0, 1.5, V).astype(np.float32)
    p = OA.softmax64(row, temperature, top_k)
    order = np.argsort(-p)
    parents = [-1, -1, -1]
    logits = np.broadcast_to(np.stack([row] + [rng.normal(0, 1.5, V).astype(np.float32) for _ in parents]), (B, 4, V))
    tokens = np.broadcast_to(np.array([0, order[1], order[7], order[20]], np.int64), (B, 4))   # 2nd, 8th, and one outside
    n, out, kt, _ = _device_walk(ctx, logits, tokens, [-1, 0, 0, 0], 1, temperature, top_k, seed=3, offset=0)
    hist = np.bincount(out[:, 0], minlength=V) / B
    assert np.abs(hist - p).max() < 4.0 * np.sqrt(p.max() * (1 - p.max()) / B) + 1e-3
    assert hist[p == 0].sum() == 0.0
    # a child is taken exactly when its token is the committed one
    took = kt[:, 1]
    assert np.all((took == 1) == ((out[:, 0] == order[1]) & (n == 1)))
    assert np.all(took != 3)                        # the child outside the top-k set is never accepted


def test_tree_engine_stochastic_rounds():
    """`TreeSpecEngine(temperature > 0)`: the replayed graph commits what eager rounds commit (same seed), different
    seeds part ways, and every committed token lies in the target's top-k set given the tokens before it."""
    import versenext_b200 as vn
    cfg = OM.small_config(tie_weights=False, init_std=0.2)
    d_cfg = OM.small_config(n_layer=1, tie_weights=False, init_std=0.2)
    t_sd = OM.init_state_dict(cfg, seed=101, gate_std=1.0)
    d_sd = OM.init_state_dict(d_cfg, seed=102, gate_std=1.0)
    d_sd["tok_emb.weight"], d_sd["head.weight"] = t_sd["tok_emb.weight"], t_sd["head.weight"]
    for n in list(d_sd):          # a draft that often agrees: the target's first block, perturbed
        if n.startswith("blocks.0.") and not n.endswith("norm1.weight") and not n.endswith("norm2.weight"):
            d_sd[n] = (t_sd[n] + 0.15 * d_sd[n]).astype(np.float32)

    def build(c, sd):
        kw = c.to_dict()
        kw.pop("init_std")
        m = vn.VerseNexLM(**kw)
        m.load_state_dict(sd)
        return m
    t, d = build(cfg, t_sd), build(d_cfg, d_sd)
    prompts = np.random.default_rng(4).integers(0, cfg.vocab_size, (3, 12))
    runs = {}
    for name, graph, seed in (("eager", False, 9), ("graph", True, 9), ("other", True, 10)):
        eng = vn.TreeSpecEngine(t, d, CFG3_TREE, max_batch=3, max_seq=160, max_new_tokens=64, graph=graph,
                                temperature=0.9, top_k=6, seed=seed)
        toks, st = eng.generate(prompts, 40)
        runs[name] = toks[:, :52]
        assert st["rounds"] < 40                    # more than one token per round on average
    np.testing.assert_array_equal(runs["eager"], runs["graph"])
    assert not np.array_equal(runs["graph"], runs["other"])
    seq = runs["graph"]
    lg = OM.forward(t_sd, cfg, seq)[0]
    for b in range(3):
        for i in range(12, seq.shape[1]):
            kept = OA.scaled_logits(lg[b, i - 1], 0.9, 7) > -np.inf     # one more than top_k: a near-tie at the cut
            assert kept[seq[b, i]], (b, i)
    with pytest.raises(ValueError):
        vn.TreeSpecEngine(t, d, CFG3_TREE, max_batch=1, max_seq=64, temperature=0.9, top_k=0)
