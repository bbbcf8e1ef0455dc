"""Acceptance / sampling kernels against the CPU oracle (through the C ABI)."""

import numpy as np
import pytest

from oracle import accept as OA
from oracle import philox as OP

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import versenext_b200 as vn
    return vn.Context.get(0)


def make(rng, B, k, V, sigma_q=2.0, sigma_d=0.5):
    q = rng.normal(0, sigma_q, (B, k, V)).astype(np.float32)
    p = np.empty((B, k + 1, V), np.float32)
    p[:, :k] = q + rng.normal(0, sigma_d, (B, k, V)).astype(np.float32)
    p[:, k] = rng.normal(0, sigma_q, (B, V)).astype(np.float32)
    draft = np.empty((B, k), np.int64)
    for b in range(B):
        for i in range(k):
            draft[b, i] = OA._inverse_cdf(OA.softmax64(q[b, i]), float(rng.random()))
    return p, q, draft


def run(ctx, p, q, draft, **kw):
    from versenext_b200 import sampling
    n, t = sampling.accept(ctx, p, q, draft, **kw)
    return n.numpy(), t.numpy()


def test_philox_matches_oracle(ctx):
    from versenext_b200 import sampling
    for purpose in (0, 1):
        got = sampling.philox_uniforms(ctx, 1234, 7, 9, 5, purpose)
        want = OP.uniform(1234, 7, np.arange(9)[:, None], np.arange(5)[None, :], purpose)
        np.testing.assert_array_equal(got, want)
    got = sampling.philox_uniforms(ctx, (5 << 32) | 17, 0, 3, 2, 0)
    np.testing.assert_array_equal(got, OP.uniform((5 << 32) | 17, 0, np.arange(3)[:, None], np.arange(2)[None, :], 0))


@pytest.mark.parametrize("V", [7, 256, 1000, 4096, 4099, 12290])
@pytest.mark.parametrize("k", [1, 4, 6])
def test_greedy_matches_oracle(ctx, V, k):
    rng = np.random.default_rng(V * 10 + k)
    B = 5
    p, q, draft = make(rng, B, k, V)
    pred = np.argmax(p, -1)
    draft[0] = pred[0, :k]                      # all accepted
    draft[1, 0] = (pred[1, 0] + 1) % V          # first rejected
    if k > 1:
        draft[2, :k - 1] = pred[2, :k - 1]      # last rejected
        draft[2, k - 1] = (pred[2, k - 1] + 1) % V
    for bonus in (True, False):
        pp = p if bonus else np.ascontiguousarray(p[:, :k])
        n, t = run(ctx, pp, None, draft, temperature=0.0, bonus=bonus)
        wn, wt = OA.accept_greedy(p, draft, bonus)
        np.testing.assert_array_equal(n, wn)
        np.testing.assert_array_equal(t, wt)


def test_greedy_ties_take_lowest_index(ctx):
    p = np.zeros((2, 2, 9000), np.float32)
    p[0, 0, [17, 4500, 8999]] = 3.0
    p[0, 1, [8191, 8192]] = 1.0
    p[1, 0, 4096] = 2.0
    p[1, 0, 4095] = 2.0
    draft = np.array([[17], [4095]], np.int64)
    n, t = run(ctx, p, None, draft, temperature=0.0, bonus=True)
    np.testing.assert_array_equal(n, [1, 1])
    np.testing.assert_array_equal(t, [[17, 8191], [4095, 0]])


@pytest.mark.parametrize("V,k,B", [(50, 2, 16), (1000, 4, 12), (4096, 4, 8), (8195, 3, 8), (20001, 4, 6)])
@pytest.mark.parametrize("temperature", [1.0, 0.7])
def test_stochastic_matches_oracle_injected_uniforms(ctx, V, k, B, temperature):
    rng = np.random.default_rng(V + k)
    p, q, draft = make(rng, B, k, V)
    ua = rng.random((B, k)).astype(np.float32)
    us = rng.random((B, k + 1)).astype(np.float32)
    ua[0] = 0.0          # row 0 accepts everything -> bonus path
    ua[1, 0] = 0.99999   # row 1 (almost surely) rejects at once
    n, t = run(ctx, p, q, draft, u_accept=ua, u_sample=us, temperature=temperature)
    wn, wt = OA.accept(p, q, draft, ua, us, temperature, 0)
    np.testing.assert_array_equal(n, wn)
    np.testing.assert_array_equal(t, wt)
    assert n[0] == k and t[0, k] >= 0


def test_stochastic_philox_matches_oracle(ctx):
    rng = np.random.default_rng(3)
    B, k, V = 10, 4, 6000
    p, q, draft = make(rng, B, k, V)
    for offset in (0, 5):
        n, t = run(ctx, p, q, draft, seed=1234, offset=offset, temperature=1.0)
        ua, us = OP.uniforms_for_call(1234, offset, B, k)
        wn, wt = OA.accept(p, q, draft, ua, us, 1.0, 0)
        np.testing.assert_array_equal(n, wn)
        np.testing.assert_array_equal(t, wt)


def test_no_bonus_and_deterministic_proposals(ctx):
    rng = np.random.default_rng(4)
    B, k, V = 12, 3, 3000
    p, q, draft = make(rng, B, k, V, sigma_q=3.0)
    draft[:, 0] = np.argmax(p[:, 0], -1)     # likely accepted under a point-mass q
    ua = rng.random((B, k)).astype(np.float32)
    us = rng.random((B, k + 1)).astype(np.float32)
    n, t = run(ctx, p, None, draft, u_accept=ua, u_sample=us, temperature=1.0)
    wn, wt = OA.accept(p, None, draft, ua, us, 1.0, 0)
    np.testing.assert_array_equal(n, wn)
    np.testing.assert_array_equal(t, wt)
    pk = np.ascontiguousarray(p[:, :k])
    ua[:] = 0.0
    n, t = run(ctx, pk, q, draft, u_accept=ua, u_sample=us, temperature=1.0, bonus=False)
    wn, wt = OA.accept(pk, q, draft, ua, us, 1.0, 0, bonus=False)
    np.testing.assert_array_equal(n, wn)
    np.testing.assert_array_equal(t, wt)
    assert np.all(t[:, k] == -1)


@pytest.mark.parametrize("V,top_k", [(300, 5), (5000, 50), (33000, 50), (5000, 1), (64, 200)])
def test_topk_matches_oracle(ctx, V, top_k):
    rng = np.random.default_rng(V + top_k)
    B, k = 8, 4
    p, q, draft = make(rng, B, k, V)
    # draft tokens drawn from the draft's own top-k distribution, as a real draft model does
    for b in range(B):
        for i in range(k):
            draft[b, i] = OA._inverse_cdf(OA.softmax64(q[b, i], 0.8, top_k), float(rng.random()))
    ua = rng.random((B, k)).astype(np.float32)
    us = rng.random((B, k + 1)).astype(np.float32)
    ua[0] = 0.0
    n, t = run(ctx, p, q, draft, u_accept=ua, u_sample=us, temperature=0.8, top_k=top_k)
    wn, wt = OA.accept(p, q, draft, ua, us, 0.8, top_k)
    np.testing.assert_array_equal(n, wn)
    np.testing.assert_array_equal(t, wt)


def test_topk_keeps_ties(ctx):
    from versenext_b200 import sampling
    V = 5000
    lg = np.full((1, V), -5.0, np.float32)
    lg[0, [10, 20, 30, 40]] = 2.0   # four-way tie at the top, top_k = 2 keeps all four
    seen = set()
    for s in range(40):
        u = np.array([[(s + 0.5) / 40]], np.float32)
        tok = sampling.sample(ctx, lg, temperature=1.0, top_k=2, uniforms=u).numpy()
        want = OA._inverse_cdf(OA.softmax64(lg[0], 1.0, 2), float(u[0, 0]))
        assert tok[0] == want
        seen.add(int(tok[0]))
    assert seen == {10, 20, 30, 40}


def test_plain_sampling_chi_square(ctx):
    from versenext_b200 import sampling
    rng = np.random.default_rng(8)
    V, R = 40, 20000
    row = rng.normal(0, 1.5, V).astype(np.float32)
    lg = np.broadcast_to(row, (R, V)).copy()
    tok = sampling.sample(ctx, lg, temperature=1.0, seed=99, offset=1).numpy()
    want = OA.softmax64(row)
    cnt = np.bincount(tok, minlength=V)
    chi2 = np.sum((cnt - R * want) ** 2 / (R * want))
    assert chi2 < 90.0   # 39 dof: p ~ 1e-5


def test_speculative_output_distribution_chi_square(ctx):
    """First committed token is distributed as p_0 whatever the draft distribution is."""
    rng = np.random.default_rng(9)
    V, k, B = 30, 3, 20000
    p_row = rng.normal(0, 1.5, (k + 1, V)).astype(np.float32)
    q_row = (p_row[:k] + rng.normal(0, 1.0, (k, V))).astype(np.float32)
    p = np.broadcast_to(p_row, (B, k + 1, V)).copy()
    q = np.broadcast_to(q_row, (B, k, V)).copy()
    qp = OA.softmax64(q_row)
    draft = np.stack([rng.choice(V, size=B, p=qp[i]) for i in range(k)], axis=1).astype(np.int64)
    n, t = run(ctx, p, q, draft, seed=4321, offset=0, temperature=1.0)
    want = OA.softmax64(p_row[0])
    cnt = np.bincount(t[:, 0], minlength=V)
    chi2 = np.sum((cnt - B * want) ** 2 / (B * want))
    assert chi2 < 75.0   # 29 dof
    # acceptance rate of position 0 equals sum(min(p, q))
    rate = np.mean(n >= 1)
    assert abs(rate - np.minimum(want, qp[0]).sum()) < 0.02


def test_cfg2_shape_reduced_batch_matches_oracle(ctx):
    """Full vocabulary 248320, k = 4, 6 sequences: bit-exact decisions and tokens."""
    p, q, draft = OA.make_cfg2_inputs(batch=6, k=4, vocab=248320, seed=1234)
    n, t = run(ctx, p, q, draft, seed=1234, offset=0, temperature=1.0)
    ua, us = OP.uniforms_for_call(1234, 0, 6, 4)
    wn, wt = OA.accept(p, q, draft, ua, us, 1.0, 0)
    np.testing.assert_array_equal(n, wn)
    np.testing.assert_array_equal(t, wt)


def test_cfg2_full_size_properties(ctx):
    """B = 64, k = 4, V = 248320: determinism, padding, greedy == argmax, acceptance rate sane."""
    rng = np.random.default_rng(1234)
    B, k, V = 64, 4, 248320
    q = rng.standard_normal((B, k, V), dtype=np.float32) * 2.0
    p = np.empty((B, k + 1, V), np.float32)
    p[:, :k] = q + rng.standard_normal((B, k, V), dtype=np.float32) * 0.5
    p[:, k] = rng.standard_normal((B, V), dtype=np.float32) * 2.0
    draft = np.argmax(q + rng.gumbel(size=q.shape).astype(np.float32), -1).astype(np.int64)  # samples from softmax(q)
    import versenext_b200 as vn
    pd, qd, dd = ctx.from_numpy(p), ctx.from_numpy(q), ctx.from_numpy(draft)
    n1, t1 = run(ctx, pd, qd, dd, seed=1234, temperature=1.0)
    n2, t2 = run(ctx, pd, qd, dd, seed=1234, temperature=1.0)
    np.testing.assert_array_equal(n1, n2)
    np.testing.assert_array_equal(t1, t2)
    assert np.all((n1 >= 0) & (n1 <= k))
    for b in range(B):
        assert np.all(t1[b, :n1[b]] == draft[b, :n1[b]])
        assert 0 <= t1[b, n1[b]] < V
        assert np.all(t1[b, n1[b] + 1:] == -1)
    assert 0.3 < n1.mean() / k < 1.0
    ng, tg = run(ctx, pd, None, dd, temperature=0.0)
    wn, wt = OA.accept_greedy(p, draft, True)
    np.testing.assert_array_equal(ng, wn)
    np.testing.assert_array_equal(tg, wt)


def test_invalid_arguments_raise(ctx):
    p = np.zeros((2, 3, 10), np.float32)
    d = np.zeros((2, 2), np.int64)
    from versenext_b200 import sampling
    with pytest.raises(ValueError):
        sampling.accept(ctx, p, None, np.zeros((2, 40), np.int64), temperature=0.0, shape=(2, 40, 10))
    with pytest.raises(ValueError):
        sampling.accept(ctx, p, None, d, temperature=1.0, top_k=5000, shape=(2, 2, 100000))


def _draft_from_topk(rng, q, temperature, top_k):
    B, k, _ = q.shape
    d = np.empty((B, k), np.int64)
    for b in range(B):
        for i in range(k):
            d[b, i] = OA._inverse_cdf(OA.softmax64(q[b, i], temperature, top_k), float(rng.random()))
    return d


def test_topk_full_vocabulary_matches_oracle(ctx):
    """The acceptance path a speculative round runs -- top-k 50 at temperature 0.8 over the whole vocabulary of
    248,320 -- against the oracle, decisions and tokens bit-exact.  Rows are shaped to walk every branch of the
    select: plain logits (bound pass suffices), an adversarial order plus heavy ties above the bound (the
    candidate buffer overflows and the radix select takes over), ties exactly at the k-th value (all kept), a row
    of few distinct values."""
    rng = np.random.default_rng(50)
    B, k, V, top_k, T = 5, 4, 248320, 50, 0.8
    p, q, _ = make(rng, B, k, V)
    # (1) sixty large distinct values packed into the first 60 positions (they fall to a handful of the bound
    # pass's thread groups) and 1,100 entries tied at a value above the bound but below the k-th largest
    p[1, 0, :60] = 20.0 + np.arange(60, dtype=np.float32) * 0.25
    p[1, 0, rng.choice(np.arange(100, 12000), 1100, replace=False)] = 9.5
    # (2) thirty distinct values on top, then forty entries tied at the value where the k-th falls
    p[2, 1, rng.choice(V, 30, replace=False)] = 15.0 + np.arange(30, dtype=np.float32)
    p[2, 1, rng.choice(np.arange(5000, 240000), 40, replace=False)] = 12.0
    # (3) the same on a draft row: q's support is what decides q(x)
    q[3, 2, rng.choice(V, 200, replace=False)] = 11.0
    # (4) a row with three distinct values only
    p[4, 3] = np.where(rng.random(V) < 0.001, 2.0, np.where(rng.random(V) < 0.5, -1.0, -3.0)).astype(np.float32)
    draft = _draft_from_topk(rng, q, T, top_k)
    ua = rng.random((B, k)).astype(np.float32)
    us = rng.random((B, k + 1)).astype(np.float32)
    # proposals equal to the target's arg-max with u = 0 are always accepted: sequence 0 runs through to the bonus
    # token, the others reach the position of their shaped row
    for b, upto in ((0, k), (2, 1), (3, 2), (4, 3)):
        draft[b, :upto] = np.argmax(p[b, :upto], -1)
        ua[b, :upto] = 0.0
    n, t = run(ctx, p, q, draft, u_accept=ua, u_sample=us, temperature=T, top_k=top_k)
    wn, wt = OA.accept(p, q, draft, ua, us, T, top_k)
    np.testing.assert_array_equal(n, wn)
    np.testing.assert_array_equal(t, wt)
    # the shaped rows were really used by at least one decision each
    kept1 = np.count_nonzero(p[1, 0] / np.float32(T) >= np.sort(p[1, 0] / np.float32(T))[-top_k])
    kept2 = np.count_nonzero(p[2, 1] >= np.sort(p[2, 1])[-top_k])
    assert kept1 == 50 and kept2 == 70
    assert wn[0] == k and wn[2] >= 1 and wn[3] >= 2 and wn[4] >= 3
    # Philox-driven call on the same rows
    n, t = run(ctx, p, q, draft, seed=77, offset=3, temperature=T, top_k=top_k)
    ua2, us2 = OP.uniforms_for_call(77, 3, B, k)
    wn, wt = OA.accept(p, q, draft, ua2, us2, T, top_k)
    np.testing.assert_array_equal(n, wn)
    np.testing.assert_array_equal(t, wt)


def test_cfg2_full_batch_row_subset_matches_oracle(ctx):
    """B = 64, k = 4, V = 248,320 (the isolated acceptance workload at full size) with Philox uniforms: the
    device call runs on all 64 sequences, the oracle re-computes a subset of them (a sequence's result depends
    on its own rows and its own Philox row index only)."""
    rng = np.random.default_rng(1234)
    B, k, V = 64, 4, 248320
    q = rng.standard_normal((B, k, V), dtype=np.float32) * 2.0
    p = np.empty((B, k + 1, V), np.float32)
    p[:, :k] = q + rng.standard_normal((B, k, V), dtype=np.float32) * 0.5
    p[:, k] = rng.standard_normal((B, V), dtype=np.float32) * 2.0
    draft = np.argmax(q + rng.gumbel(size=q.shape).astype(np.float32), -1).astype(np.int64)
    n, t = run(ctx, p, q, draft, seed=1234, offset=0, temperature=1.0)
    ua, us = OP.uniforms_for_call(1234, 0, B, k)
    rows = [0, 1, 17, 31, 32, 50, 63]
    wn, wt = OA.accept(p[rows], q[rows], draft[rows], ua[rows], us[rows], 1.0, 0)
    np.testing.assert_array_equal(n[rows], wn)
    np.testing.assert_array_equal(t[rows], wt)


def test_sampling_distribution_equals_the_reference_samplers(ctx, golden):
    """The distribution `vn_sample` draws from, read off through injected uniforms, against the probability
    vectors recorded from the reference's `Sampler.sample` (sampler.py:86-138; ties at the k-th value kept):
    for every kept token, uniforms just inside both ends and in the middle of its CDF interval must return it,
    so every interval edge sits within a twentieth of the token's probability of the reference's."""
    from versenext_b200 import sampling
    g = golden("sampling_reference.npz")
    rows = g["rows"]
    for ci, (T, k) in enumerate(zip(g["temperature"], g["top_k"])):
        for ri in range(rows.shape[0]):
            ref = g[f"sampler_c{ci}_r{ri}"]
            kept = np.flatnonzero(ref > 0)
            cdf = np.cumsum(ref[kept])
            lo = np.concatenate([[0.0], cdf[:-1]]) / cdf[-1]
            hi = cdf / cdf[-1]
            wide = (hi - lo) > 2e-5                   # float32 uniforms cannot address much narrower intervals
            toks, us = [], []
            for frac in (0.05, 0.5, 0.95):
                us.append(lo[wide] + frac * (hi[wide] - lo[wide]))
                toks.append(kept[wide])
            us, toks = np.concatenate(us).astype(np.float32), np.concatenate(toks)
            ok = (us > 0) & (us < 1)
            us, toks = us[ok], toks[ok]
            lg = np.broadcast_to(rows[ri], (us.size, rows.shape[1])).copy()
            got = sampling.sample(ctx, lg, temperature=float(T), top_k=int(k), uniforms=us).numpy()
            np.testing.assert_array_equal(got, toks, err_msg=f"case {ci} row {ri}")
