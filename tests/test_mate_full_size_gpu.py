"""Full-size properties of the mate-shaped target (D=1024, 20 layers: 5 MoD + 15 TriSparse, V=248320, bf16).

The CPU oracle cannot run this size in seconds, so these tests check relations that hold at any size:
tree verification against per-path chain forwards, accepted-path commit against a fresh prefill, determinism of
the batched speculative engine, and the weight-only quantised variants against the bf16 model they came from.
Weights are seeded N(0, 0.02) (synthetic), prompts are uniform random ids, as in the benchmark configurations.
"""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

V = 248320
# 16-node tree: four children of the context, then two per node, then two per node of the first four
PARENTS = [-1, -1, -1, -1, 0, 0, 1, 1, 4, 4, 5, 5, 6, 6, 7, 7]


def rel_err(a, b):
    return float(np.max(np.abs(a - b)) / np.max(np.abs(b)))


def path_of(node):
    p = []
    while node >= 0:
        p.append(node)
        node = PARENTS[node]
    return p[::-1]


@pytest.fixture(scope="module")
def mate():
    import versenext_b200 as vn
    from versenext_b200 import synthetic
    kw = synthetic.mate_kwargs()
    m = vn.VerseNexLM(dtype="bf16", **kw)
    synthetic.load_random(m, kw, seed=3)
    return m, kw


def test_parameter_count_and_bytes(mate):
    from versenext_b200 import synthetic
    m, kw = mate
    assert synthetic.param_count(kw) == 1_107_375_164          # the figure the roofline bytes are computed from


def test_tree_verification_equals_chain_forward_full_size(mate):
    """Config 3 shape: B=8, a cache of 2048 tokens, 16 tree nodes with an ancestor mask.  The logits of a node
    must equal the last-position logits of a plain chain forward over its root-to-node path."""
    m, kw = mate
    rng = np.random.default_rng(3)
    B, T = 8, 2048
    prompt = rng.integers(0, V, (B, T))
    cache = m.new_cache(B, T + 64)
    for lo in range(0, T, 256):                                   # chunked prefill on the same cache
        m.forward_cached(prompt[:, lo:lo + 256], cache, last_only=True)
        cache.commit(256, np.full(B, 256, np.int32))
    assert list(cache.per_seq_lens[:B]) == [T] * B
    nodes = rng.integers(0, V, (B, 16))
    tree = m.forward_cached(nodes, cache, parents=PARENTS).numpy()          # (B, 16, V); nothing committed
    assert np.isfinite(tree).all()
    for leaf in (8, 11, 15, 3):
        path = path_of(leaf)
        chain = m.forward_cached(nodes[:, path], cache).numpy()             # same uncommitted slots, causal mask
        for i, node in enumerate(path):
            assert rel_err(tree[:, node], chain[:, i]) < 2e-2
        assert (tree[:, leaf].argmax(-1) == chain[:, -1].argmax(-1)).mean() >= 0.75
    # siblings see different tokens only at their own position: their logits must differ
    assert np.abs(tree[:, 8] - tree[:, 9]).max() > 0


def test_commit_of_accepted_path_matches_fresh_prefill(mate):
    """Keep a root-to-node path of a verified tree (in-place compaction, the rest rolled back): the next-token
    logits equal those of a cache that was prefilled with prompt + path directly."""
    m, kw = mate
    rng = np.random.default_rng(33)
    B, T = 4, 300
    prompt = rng.integers(0, V, (B, T))
    nodes = rng.integers(0, V, (B, 16))
    nxt = rng.integers(0, V, (B, 1))
    path = path_of(13)                                            # 1 -> 6 -> 13
    cache = m.new_cache(B, 512)
    m.forward_cached(prompt, cache, last_only=True)
    cache.commit(T, np.full(B, T, np.int32))
    m.forward_cached(nodes, cache, parents=PARENTS, last_only=True)
    keep = np.tile(np.asarray(path, np.int32), (B, 1))
    cache.commit(16, np.full(B, len(path), np.int32), keep_idx=keep)
    assert list(cache.per_seq_lens[:B]) == [T + len(path)] * B
    got = m.forward_cached(nxt, cache).numpy()
    fresh = m.new_cache(B, 512)
    full = np.concatenate([prompt, nodes[:, path]], axis=1)
    m.forward_cached(full, fresh, last_only=True)
    fresh.commit(full.shape[1], np.full(B, full.shape[1], np.int32))
    want = m.forward_cached(nxt, fresh).numpy()
    assert rel_err(got, want) < 2e-2


def test_speculative_engine_full_size_is_deterministic_and_consistent(mate):
    """Config 4 shape at one GPU (32 requests, 512-token prompts, k=4, T=0.8, top-k 50, 2-layer draft): the same
    seed gives the same tokens eagerly and from the replayed graph; every round commits 1..k+1 tokens per request."""
    import versenext_b200 as vn
    from versenext_b200 import synthetic
    m, kw = mate
    dkw = synthetic.draft_kwargs()
    d = vn.VerseNexLM(dtype="bf16", **dkw)
    synthetic.load_random(d, dkw, seed=5)
    prompts = np.random.default_rng(4).integers(0, V, (32, 512))
    outs = []
    for graph in (True, False):
        eng = vn.SpecEngine(m, d, max_batch=32, max_seq=640, k=4, temperature=0.8, top_k=50, seed=4, graph=graph)
        eng.prefill(prompts)
        before = eng.counts().copy()
        per_round = []
        for _ in range(6):
            eng.step()
            now = eng.counts().copy()
            per_round.append(now - before)
            before = now
        per_round = np.stack(per_round)
        assert per_round.min() >= 1 and per_round.max() <= 5
        toks = eng.tokens()
        assert all((0 <= np.asarray(t)).all() and (np.asarray(t) < V).all() for t in toks)
        outs.append([np.asarray(t).copy() for t in toks])
    for a, b in zip(*outs):
        np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("scheme,tol", [("int8", 0.05), ("int4g128", 0.25)])
def test_quantised_mate_tracks_the_bf16_model(scheme, tol):
    """Config 5's target variants on one GPU: quantise the loaded bf16 model in place and compare the verify
    logits (7 positions, k=6) with those of the dense model; the weight bytes shrink as the scheme says."""
    import versenext_b200 as vn
    from versenext_b200 import synthetic
    kw = synthetic.mate_kwargs()
    m = vn.VerseNexLM(dtype="bf16", **kw)
    synthetic.load_random(m, kw, seed=3)
    rng = np.random.default_rng(5)
    B, T = 4, 96
    prompt = rng.integers(0, V, (B, T))
    nxt = rng.integers(0, V, (B, 7))

    def run():
        cache = m.new_cache(B, 128)
        m.forward_cached(prompt, cache, last_only=True)
        cache.commit(T, np.full(B, T, np.int32))
        return m.forward_cached(nxt, cache).numpy()

    dense = run()
    dense_bytes = m.param_bytes()
    m.quantize(scheme)
    quant = run()
    assert np.isfinite(quant).all()
    assert rel_err(quant, dense) < tol
    per_weight = {"int8": 1.0, "int4g128": 0.5 + 2.0 / 128}[scheme]
    linear = 1_104_711_680                                        # linear parameters incl. the un-tied head copy
    expect = linear * per_weight
    assert 0.9 * expect < m.param_bytes() - 254_279_680 * 2 < 1.15 * expect + 64e6   # embedding stays bf16
    assert m.param_bytes() < dense_bytes
