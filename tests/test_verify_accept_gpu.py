"""`vn_verify_accept`: target forward + LM head + acceptance in one call, with the head fused into the top-k
selection (the logits never reach memory) -- against the stored-logits route (forward, then `vn_accept_strided`,
itself checked against the oracle in test_accept_gpu.py) and against the oracle directly."""

import ctypes as C

import numpy as np
import pytest

from oracle import accept as OA
from oracle import model as OM

pytestmark = pytest.mark.gpu


def _ptr(a):
    return C.c_void_p(a.ptr) if a is not None else None


def _model(vocab, seed, ties=0, tie_scale=3.0):
    import versenext_b200 as vn
    cfg = OM.mate_config(vocab_size=vocab, dim=128, n_layer=2, n_head=2, n_kv_head=1, window_size=32,
                         num_global_tokens=8, max_seq_len=256, init_std=0.08, num_dense_parts=2,
                         num_experts_per_part=2, top_k=1, expert_hidden=128, mlp_hidden_multiple=2)
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=seed, gate_std=1.0).items()}
    if ties:
        # `ties` vocabulary columns behind the first 8,192 share one embedding row: their logits are equal in every
        # row, and where that value lies above the row's bound the candidate list of the fused head overflows
        emb = sd["tok_emb.weight"].copy()
        emb[8192:8192 + ties] = OM.bf16_round(emb[8192] * np.float32(tie_scale))
        sd["tok_emb.weight"] = emb
    kw = cfg.to_dict()
    kw.pop("init_std")
    m = vn.VerseNexLM(dtype="bf16", **kw)
    m.load_state_dict(sd)
    return cfg, sd, m


def _call(m, cache, tokens, k, q_logits, draft, ua, us, temperature, top_k, bonus, scratch, q_lists=None, B_stride=None):
    ctx = m.ctx
    B, T = tokens.shape
    out_len, out_tok = ctx.zeros((B,), np.int32), ctx.zeros((B, k + 1), np.int64)
    V = m.vocab_size
    ctx._check(ctx.lib.vn_verify_accept(
        m.handle, cache.handle, _ptr(tokens), B, T, k, _ptr(q_lists), 1, B,
        _ptr(q_logits), k * V, V, _ptr(draft), _ptr(ua), _ptr(us), 11, 2, float(temperature), int(top_k), int(bonus),
        _ptr(scratch), _ptr(out_len), _ptr(out_tok)))
    return out_len.numpy(), out_tok.numpy()


def _setup(m, rng, B, k, T0=40):
    ctx = m.ctx
    V = m.vocab_size
    cache = m.new_cache(B, 128)
    m.forward_cached(rng.integers(0, V, (B, T0)), cache, want_logits=False, want_hidden=True, last_only=True)
    cache.commit(T0, np.full(B, T0, np.int32))
    tokens = ctx.from_numpy(rng.integers(0, V, (B, k + 1)).astype(np.int64))
    return cache, tokens


@pytest.mark.parametrize("vocab,ties", [(2048, 0), (16384, 0), (16384, 5000)])
@pytest.mark.parametrize("injected", [True, False])
def test_fused_head_equals_stored_logits_route(vocab, ties, injected, monkeypatch):
    rng = np.random.default_rng(vocab + ties)
    cfg, sd, m = _model(vocab, seed=5, ties=ties)
    ctx = m.ctx
    B, k, top_k, T = 6, 3, 20, 0.8
    cache, tokens = _setup(m, rng, B, k)
    V = vocab
    q = ctx.from_numpy(rng.normal(0, 2.0, (B, k, V)).astype(np.float32))
    # proposals: mostly the target's own arg-max (so that later positions are reached), some random
    lg = m.forward_cached(tokens, cache).numpy()
    draft = np.argmax(lg[:, :k], -1).astype(np.int64)
    draft[1, 1] = rng.integers(0, V)
    draft[2, 0] = rng.integers(0, V)
    dd = ctx.from_numpy(draft)
    ua = ctx.from_numpy((rng.random((B, k)) * 0.5).astype(np.float32)) if injected else None
    us = ctx.from_numpy(rng.random((B, k + 1)).astype(np.float32)) if injected else None
    scratch = ctx.empty((B, k + 1, V), np.float32)
    monkeypatch.setenv("VN_K1", "0")
    want = _call(m, cache, tokens, k, q, dd, ua, us, T, top_k, True, scratch)
    monkeypatch.setenv("VN_K1", "1")
    l0 = ctx.launch_count()
    got = _call(m, cache, tokens, k, q, dd, ua, us, T, top_k, True, scratch)
    np.testing.assert_array_equal(got[0], want[0])
    np.testing.assert_array_equal(got[1], want[1])
    assert np.all(got[1][np.arange(B), got[0]] >= 0)
    # and against the oracle on the device's own logits (the tie construction keeps more than the lists can hold
    # in some rows, where the device truncates: those are compared with the stored-logits route only)
    if not ties and injected:
        wn, wt = OA.accept(lg, q.numpy(), draft, ua.numpy(), us.numpy(), T, top_k)
        np.testing.assert_array_equal(got[0], wn)
        np.testing.assert_array_equal(got[1], wt)
    m.check()


def test_fused_head_without_draft_logits_and_without_bonus():
    rng = np.random.default_rng(3)
    cfg, sd, m = _model(4096, seed=9)
    ctx = m.ctx
    B, k, top_k, T = 5, 4, 10, 1.1
    cache, tokens = _setup(m, rng, B, k)
    lg = m.forward_cached(tokens, cache).numpy()
    draft = np.argmax(lg[:, :k], -1).astype(np.int64)
    draft[3, 2] = 17
    ua = rng.random((B, k)).astype(np.float32) * 0.2
    us = rng.random((B, k + 1)).astype(np.float32)
    scratch = ctx.empty((B, k + 1, 4096), np.float32)
    # point-mass proposals (no q), bonus token
    got = _call(m, cache, tokens, k, None, ctx.from_numpy(draft), ctx.from_numpy(ua), ctx.from_numpy(us), T, top_k, True,
                scratch)
    wn, wt = OA.accept(lg, None, draft, ua, us, T, top_k)
    np.testing.assert_array_equal(got[0], wn)
    np.testing.assert_array_equal(got[1], wt)
    # no bonus: T = k positions
    tok_k = ctx.from_numpy(tokens.numpy()[:, :k].copy())
    got = _call(m, cache, tok_k, k, None, ctx.from_numpy(draft), ctx.from_numpy(ua), ctx.from_numpy(us), T, top_k, False,
                scratch)
    wn, wt = OA.accept(lg[:, :k], None, draft, ua, us, T, top_k, bonus=False)
    np.testing.assert_array_equal(got[0], wn)
    np.testing.assert_array_equal(got[1], wt)
    with pytest.raises(ValueError):
        _call(m, cache, tokens, k - 1, None, ctx.from_numpy(draft), None, None, T, top_k, True, scratch)


def test_kept_lists_of_the_draft_rows_are_reused():
    """`vn_sample_lists` leaves the selection it sampled from; `vn_verify_accept` reads it as q and decides exactly
    as it does from the draft rows' logits."""
    rng = np.random.default_rng(21)
    cfg, sd, m = _model(16384, seed=2)
    ctx = m.ctx
    B, k, top_k, T, V = 7, 4, 50, 0.8, 16384
    cache, tokens = _setup(m, rng, B, k)
    q = rng.normal(0, 2.0, (k, B, V)).astype(np.float32)           # step-major, as a draft model produces them
    qd = ctx.from_numpy(q)
    rec = int(ctx.lib.vn_topk_row_bytes())
    lists = ctx.empty((k * B * rec,), np.uint8)
    steps = ctx.zeros((k, B), np.int64)
    for i in range(k):
        ctx._check(ctx.lib.vn_sample_lists(ctx.handle, _ptr(qd[i]), V, B, V, T, top_k, None, 5, 0, i, 2, _ptr(steps[i]),
                                           C.c_void_p(lists.ptr + i * B * rec)))
        want = OA_sample(q[i], T, top_k, 5, i)
        np.testing.assert_array_equal(steps[i].numpy(), want)
    draft = np.ascontiguousarray(steps.numpy().T)
    dd = ctx.from_numpy(draft)
    scratch = ctx.empty((B, k + 1, V), np.float32)
    out_len, out_tok = ctx.zeros((B,), np.int32), ctx.zeros((B, k + 1), np.int64)

    def run(q_lists, q_logits):
        ctx._check(ctx.lib.vn_verify_accept(
            m.handle, cache.handle, _ptr(tokens), B, k + 1, k, q_lists, 1, B, q_logits, V, B * V, _ptr(dd), None, None,
            77, 1, T, top_k, 1, _ptr(scratch), _ptr(out_len), _ptr(out_tok)))
        return out_len.numpy(), out_tok.numpy()

    a = run(_ptr(lists), None)
    b = run(None, _ptr(qd))
    np.testing.assert_array_equal(a[0], b[0])
    np.testing.assert_array_equal(a[1], b[1])


def OA_sample(rows, T, top_k, seed, position):
    from oracle import philox as OP
    out = np.empty(rows.shape[0], np.int64)
    for r in range(rows.shape[0]):
        u = OP.uniform(seed, 0, r, position, 2)
        out[r] = OA._inverse_cdf(OA.softmax64(rows[r], T, top_k), float(u))
    return out


def test_draft_propose_equals_the_step_by_step_loop():
    """`vn_draft_propose`: k forwards + top-k sampling in one C call -- the same proposals, logits and kept lists as
    the loop of `vn_model_forward` (two tokens first, then one at a growing slot offset) and `vn_sample_lists`
    written out by hand; a second call on the same state repeats them (nothing was committed)."""
    import versenext_b200 as vn
    rng = np.random.default_rng(77)
    V, B, k, top_k, T = 4096, 5, 4, 12, 0.9
    cfg = OM.small_config(vocab_size=V, dim=128, n_layer=2, n_head=2, n_kv_head=2, window_size=32, num_global_tokens=8,
                          max_seq_len=256)
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=4, gate_std=1.0).items()}
    kw = cfg.to_dict()
    kw.pop("init_std")
    d = vn.VerseNexLM(dtype="bf16", **kw)
    d.load_state_dict(sd)
    ctx, lib = d.ctx, d.ctx.lib
    cache = d.new_cache(B, 128)
    d.forward_cached(rng.integers(0, V, (B, 30)), cache, want_logits=False)
    cache.commit(30, np.full(B, 30, np.int32))
    pair = ctx.from_numpy(rng.integers(0, V, (B, 2)).astype(np.int64))
    rec = int(lib.vn_topk_row_bytes())
    seed = 99

    def by_hand():
        q = ctx.zeros((k, B, V), np.float32)
        steps = ctx.zeros((k, B), np.int64)
        lists = ctx.zeros((k * B * rec,), np.uint8)
        for i in range(k):
            if i == 0:
                d.forward_cached(pair, cache, last_only=True, out_logits=q[i], slot_offset=0)
            else:
                d.forward_cached(steps[i - 1].reshape(B, 1), cache, last_only=True, out_logits=q[i], slot_offset=i + 1)
            ctx._check(lib.vn_sample_lists(ctx.handle, _ptr(q[i]), V, B, V, T, top_k, None, seed, 3, i, 2, _ptr(steps[i]),
                                           C.c_void_p(lists.ptr + i * B * rec)))
        return q.numpy(), steps.numpy(), lists.numpy()

    def one_call():
        q = ctx.zeros((k, B, V), np.float32)
        steps = ctx.zeros((k, B), np.int64)
        lists = ctx.zeros((k * B * rec,), np.uint8)
        ctx._check(lib.vn_draft_propose(d.handle, cache.handle, _ptr(pair), B, k, T, top_k, seed, 3, _ptr(q), _ptr(steps),
                                        _ptr(lists)))
        return q.numpy(), steps.numpy(), lists.numpy()

    want = by_hand()
    got = one_call()
    again = one_call()
    for a, b, c in zip(want, got, again):
        np.testing.assert_array_equal(a, b)
        np.testing.assert_array_equal(b, c)
    assert got[1].min() >= 0 and got[1].max() < V
    # the proposals are draws from the draft's own top-k distribution: every token lies in its row's kept set
    for i in range(k):
        kth = np.sort(got[0][i], axis=-1)[:, -top_k]
        assert np.all(got[0][i][np.arange(B), got[1][i]] >= kth)
    # greedy rule: arg-max proposals, no lists
    q = ctx.zeros((k, B, V), np.float32)
    steps = ctx.zeros((k, B), np.int64)
    ctx._check(lib.vn_draft_propose(d.handle, cache.handle, _ptr(pair), B, k, 0.0, 0, seed, 0, _ptr(q), _ptr(steps), None))
    np.testing.assert_array_equal(steps.numpy(), np.argmax(q.numpy(), -1))
    with pytest.raises(ValueError):
        ctx._check(lib.vn_draft_propose(d.handle, cache.handle, _ptr(pair), B, 0, T, top_k, seed, 0, _ptr(q), _ptr(steps), None))
    d.check()
