"""The CPU oracle against the fixtures produced by the real reference
(tests/golden/make_golden.py) and against published known-answer vectors."""

import numpy as np
import pytest

from oracle import accept as OA
from oracle import model as OM
from oracle import philox as OP
from oracle import quant as OQ
from oracle import spec as OS


def test_philox_known_answers():
    # Random123 kat_vectors, philox4x32-10
    kat = [
        ((0, 0, 0, 0), (0, 0), (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
        ((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2, (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
        ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
         (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)),
    ]
    for ctr, key, want in kat:
        got = OP.philox4x32_10(np.array(ctr, dtype=np.uint32), np.array(key, dtype=np.uint32))
        assert tuple(int(x) for x in got) == want


def test_philox_uniform_range_and_layout():
    ua, us = OP.uniforms_for_call(1234, 3, 5, 4)
    assert ua.shape == (5, 4) and us.shape == (5, 5)
    assert ua.dtype == np.float32 and np.all((ua >= 0) & (ua < 1))
    assert OP.uniform(1234, 3, 2, 1, 0) == ua[2, 1]
    assert OP.uniform(1234, 3, 2, 1, 1) == us[2, 1]
    assert OP.uniform(1234, 4, 2, 1, 0) != ua[2, 1]


def test_speculative_decoder_against_reference(golden):
    g = golden("spec_reference.npz")
    for ci in g["cases"]:
        p = f"c{ci}_"
        draft, logits = OS.draft_heads(g[p + "hidden"], list(g[p + "heads"]))
        np.testing.assert_array_equal(draft, g[p + "draft"])
        np.testing.assert_allclose(np.stack(logits), g[p + "draft_logits"], rtol=1e-5, atol=1e-5)
        table = g[p + "table"]

        def model_fn(ids, table=table):
            return np.broadcast_to(table[None, :ids.shape[1]], (ids.shape[0], ids.shape[1], table.shape[1]))

        mask, pred = OS.verify(g[p + "draft"], model_fn, g[p + "ctx"])
        np.testing.assert_array_equal(mask, g[p + "mask"])
        np.testing.assert_array_equal(pred, g[p + "pred"])
        toks, ok, new_ctx = OS.verify_then_commit(g[p + "draft"], model_fn, g[p + "ctx"])
        assert toks == list(g[p + "tokens"]) and ok == bool(g[p + "all_ok"])
        np.testing.assert_array_equal(new_ctx, g[p + "new_ctx"])
        # the op-level greedy rule gives the same committed tokens (no bonus)
        k, T = draft.shape[1], g[p + "ctx"].shape[1]
        acc, out = OA.accept_greedy(np.broadcast_to(table[None, T - 1:T + k], (1, k + 1, table.shape[1])),
                                    g[p + "draft"][:1], bonus=False)
        assert list(out[0][out[0] >= 0]) == toks


def test_verify_errors():
    with pytest.raises(ValueError):
        OS.verify(np.zeros((2, 4), int), lambda x: x, np.zeros((3, 5), int))
    with pytest.raises(ValueError):
        OS.verify(np.zeros((4,), int), lambda x: x, np.zeros((1, 5), int))


def _sd(g, prefix):
    return {n[len(prefix):]: g[n] for n in g.files if n.startswith(prefix)}


def test_small_model_forward_and_streams(golden):
    g = golden("model_small.npz")
    t_cfg, d_cfg = OM.small_config(), OM.small_config(n_layer=1)
    t_sd, d_sd = _sd(g, "a_t."), _sd(g, "a_d.")
    lg, _ = OM.forward(t_sd, t_cfg, g["prompt"])
    np.testing.assert_allclose(lg, g["a_logits"], rtol=1e-4, atol=2e-6)
    st = OS.generate(t_sd, t_cfg, d_sd, d_cfg, g["prompt"], 4, 128)
    np.testing.assert_array_equal(st["tokens"], g["a_spec"])
    assert st["rounds"] == int(g["a_rounds"]) and st["accepted"] == int(g["a_accepted"])


def test_small_model_nondegenerate_variant(golden):
    g = golden("model_small.npz")
    t_cfg = OM.small_config(tie_weights=False, init_std=0.2)
    d_cfg = OM.small_config(n_layer=1, tie_weights=False, init_std=0.2)
    t_sd = OM.init_state_dict(t_cfg, seed=101, gate_std=1.0)
    d_sd = OM.init_state_dict(d_cfg, seed=102, gate_std=1.0)
    d_sd["tok_emb.weight"], d_sd["head.weight"] = t_sd["tok_emb.weight"], t_sd["head.weight"]
    for n in list(d_sd):
        if n.startswith("blocks.0.") and not n.endswith("norm1.weight") and not n.endswith("norm2.weight"):
            d_sd[n] = (t_sd[n] + 0.15 * d_sd[n]).astype(np.float32)
    lg, _ = OM.forward(t_sd, t_cfg, g["prompt"])
    np.testing.assert_allclose(lg, g["b_logits"], rtol=1e-4, atol=1e-4)
    cur, _ = OS.greedy_generate(t_sd, t_cfg, g["prompt"], 96)
    np.testing.assert_array_equal(cur, g["b_greedy"])
    st = OS.generate(t_sd, t_cfg, d_sd, d_cfg, g["prompt"], 4, 96)
    np.testing.assert_array_equal(st["tokens"], g["b_spec"])
    assert st["rounds"] == int(g["b_rounds"]) and st["accepted"] == int(g["b_accepted"])


def mini_cfg(**over):
    kw = dict(vocab_size=512, dim=64, n_layer=4, n_head=4, n_kv_head=2, window_size=16,
              num_global_tokens=8, max_seq_len=128, init_std=0.1)
    kw.update(over)
    return OM.mate_config(**kw)


def test_mini_mate_model(golden):
    g = golden("model_mini.npz")
    cfg = mini_cfg()
    sd = OM.init_state_dict(cfg, seed=7, gate_std=1.0)
    toks = g["tokens"]
    lg, _ = OM.forward(sd, cfg, toks)
    np.testing.assert_allclose(lg, g["logits"], rtol=2e-4, atol=2e-4)
    cfg2 = mini_cfg(embedding_scale=False, use_alibi=True)
    lg2, _ = OM.forward(sd, cfg2, toks[:1])
    np.testing.assert_allclose(lg2, g["logits_alibi_rope"], rtol=2e-4, atol=2e-4)
    # cached continuation equals the reference's own kv_cache path
    _, cache = OM.forward(sd, cfg, toks[:, :30])
    lg3, _ = OM.forward(sd, cfg, toks[:, 30:], cache=cache)
    np.testing.assert_allclose(lg3, g["logits_incremental"], rtol=2e-4, atol=2e-4)
    np.testing.assert_allclose(lg3, g["logits"][:, 30:], rtol=2e-3, atol=2e-3)


def test_tree_equals_per_path_forward():
    cfg = mini_cfg(n_layer=2)
    sd = OM.init_state_dict(cfg, seed=9, gate_std=1.0)
    rng = np.random.default_rng(2)
    ctx = rng.integers(0, 512, (1, 20))
    parents = [-1, -1, 0, 0, 1, 2, 2, 5]
    nodes = rng.integers(0, 512, (1, len(parents)))
    _, cache = OM.forward(sd, cfg, ctx)
    lg_tree, _ = OM.forward(sd, cfg, nodes, cache=cache, parents=parents)
    for i in range(len(parents)):
        path, j = [], i
        while j >= 0:
            path.append(j)
            j = parents[j]
        path = path[::-1]
        seq = np.concatenate([ctx, nodes[:, path]], axis=1)
        lg, _ = OM.forward(sd, cfg, seq)
        np.testing.assert_allclose(lg_tree[:, i], lg[:, -1], rtol=2e-3, atol=2e-4)


def test_quant_against_reference(golden):
    g = golden("quant_reference.npz")
    q8, s8 = OQ.quantize_int8(g["w"])
    np.testing.assert_array_equal(q8, g["q8"])
    np.testing.assert_array_equal(s8, g["s8"])
    p4, s4 = OQ.quantize_int4(g["w"])
    np.testing.assert_array_equal(p4, g["p4"])
    np.testing.assert_array_equal(s4, g["s4"])
    np.testing.assert_allclose(OQ.linear_int4(g["x"], p4, s4, 64), g["y4"], rtol=1e-5, atol=1e-6)
    for qt, fn in (("int8", lambda: OQ.linear_int8(g["x"], q8, s8)),
                   ("int4", lambda: OQ.linear_int4(g["x"], p4, s4, 64))):
        y = fn() + g["bias"]
        for tag in ("1", "0", "fused"):
            np.testing.assert_allclose(y, g[f"ql_{qt}_{tag}"], rtol=1e-4, atol=1e-5)


def test_int4_g128_roundtrip():
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.02, (16, 256)).astype(np.float32)
    packed, sc = OQ.quantize_int4_g128(w)
    assert packed.shape == (16, 128) and sc.shape == (16, 2)
    np.testing.assert_array_equal(sc, OM.bf16_round(sc))
    d = OQ.dequant_int4_g128(packed, sc, 256)
    assert np.max(np.abs(d - w)) <= np.max(sc) * 0.5 + 1e-6


def test_bf16_round():
    a = np.array([1.0, 1.00390625, 1.0039062, 3.1415927, -2.5e-3, 0.0], dtype=np.float32)
    import torch
    want = torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()
    np.testing.assert_array_equal(OM.bf16_round(a), want)
    r = np.random.default_rng(0).normal(0, 1, 10000).astype(np.float32)
    np.testing.assert_array_equal(OM.bf16_round(r), torch.from_numpy(r).to(torch.bfloat16).to(torch.float32).numpy())


def test_accept_reduces_to_greedy_at_t0_and_is_distribution_preserving():
    rng = np.random.default_rng(0)
    V, k, B = 12, 3, 4000
    p_row = rng.normal(0, 1.5, (k + 1, V)).astype(np.float32)
    q_row = (p_row[:k] + rng.normal(0, 1.0, (k, V))).astype(np.float32)
    p = np.broadcast_to(p_row, (B, k + 1, V))
    q = np.broadcast_to(q_row, (B, k, V))
    qp = OA.softmax64(q_row)
    draft = np.stack([rng.choice(V, size=B, p=qp[i]) for i in range(k)], axis=1)
    ua, us = OP.uniforms_for_call(77, 0, B, k)
    acc, toks = OA.accept(p, q, draft, ua, us, 1.0, 0)
    # first emitted token is distributed as p_0 whatever q is
    first = toks[:, 0]
    want = OA.softmax64(p_row[0])
    cnt = np.bincount(first, minlength=V)
    chi2 = np.sum((cnt - B * want) ** 2 / (B * want))
    assert chi2 < 40.0  # 11 dof, p ~ 3e-5
    assert np.all(toks[np.arange(B), acc] >= 0)
    a0, t0 = OA.accept(p, q, draft, None, None, 0.0, 0)
    pred = np.argmax(p_row, -1)
    for b in range(50):
        n = 0
        while n < k and draft[b, n] == pred[n]:
            n += 1
        assert a0[b] == n and t0[b, n] == pred[n]


def test_topk_keeps_ties_and_masks_rest():
    x = np.array([[0.1, 3.0, 2.0, 2.0, -1.0, 0.5]], dtype=np.float32)
    p = OA.softmax64(x, 1.0, 2)
    assert p[0, 1] > 0 and p[0, 2] > 0 and p[0, 3] > 0 and p[0, 0] == 0 and p[0, 4] == 0
    np.testing.assert_allclose(p.sum(), 1.0)


# ---- sampling rules and the recurrent decoding path, pinned to vectors recorded from the reference ----------------
def test_sampling_probabilities_match_the_reference_samplers(golden):
    """`softmax64(x, T, top_k)` is the distribution both reference samplers draw from: `Sampler.sample`
    (threshold rule, every logit >= the k-th largest kept) on every row, `_generate_with_logits` (argpartition,
    exactly k kept) wherever the k-th largest value is not tied; with ties the latter keeps a k-subset of it."""
    from oracle import accept as OA
    g = golden("sampling_reference.npz")
    rows = g["rows"]
    for ci, (T, k) in enumerate(zip(g["temperature"], g["top_k"])):
        for ri in range(rows.shape[0]):
            mine = OA.softmax64(rows[ri], float(T), int(k))
            ref = g[f"sampler_c{ci}_r{ri}"]
            assert np.array_equal(mine > 0, ref > 0), (ci, ri)
            np.testing.assert_allclose(mine, ref, rtol=2e-5, atol=1e-9)
            gen = g[f"generate_c{ci}_r{ri}"]
            scaled = rows[ri] / np.float32(max(T, 1e-8))
            kk = min(int(k), rows.shape[1]) if k > 0 else rows.shape[1]
            kth = np.sort(scaled)[-kk]
            if np.count_nonzero(scaled >= kth) == kk:
                np.testing.assert_allclose(mine, gen, rtol=2e-5, atol=1e-9)
            else:                               # ties at the threshold: exactly k of the tied set survive
                assert np.count_nonzero(gen) == kk and np.all((gen > 0) <= (mine > 0)), (ci, ri)


@pytest.mark.parametrize("tag", ["alibi", "rope"])
def test_recurrent_path_matches_the_reference_beyond_the_window(golden, tag):
    g = golden("recurrent_reference.npz")
    cfg = (OM.small_config(tie_weights=False, init_std=0.2) if tag == "alibi" else
           OM.mate_config(vocab_size=512, dim=64, n_layer=2, n_head=4, n_kv_head=2, window_size=16,
                          num_global_tokens=8, max_seq_len=256, init_std=0.2, num_dense_parts=2,
                          num_experts_per_part=2, top_k=1, layer_pattern=["trisparse", "trisparse"],
                          embedding_scale=False))
    sd = {n[len(tag) + 1:]: g[n] for n in g.files if n.startswith(tag + ".")}
    toks = g[f"{tag}_tokens"]
    want = g[f"{tag}_recurrent_logits"]
    got, _ = OM.forward(sd, cfg, toks, recurrent=True)
    assert float(np.max(np.abs(got - want)) / np.max(np.abs(want))) < 1e-4
    if tag == "alibi":
        # the whole-sequence forward lets the ALiBi path see every earlier key; with slopes >= 1/2 a key beyond
        # the window carries a weight below e^-16, so the two rules agree far inside the tolerance while the
        # path is on (they part only past 1,024 keys, where the whole-sequence forward switches the path off)
        full, _ = OM.forward(sd, cfg, toks)
        assert float(np.max(np.abs(full - want)) / np.max(np.abs(want))) < 1e-4
    W = cfg.window_size
    out = OM.generate_greedy_recurrent(sd, cfg, toks[:, :W + 5], W + 7)
    np.testing.assert_array_equal(out, g[f"{tag}_generate"])
    eos = int(g[f"{tag}_generate"][0, W + 6])
    out = OM.generate_greedy_recurrent(sd, cfg, toks[:1, :6], 12, eos_id=eos)
    np.testing.assert_array_equal(out, g[f"{tag}_generate_eos"])


def test_delta_attention_family_against_the_reference(golden):
    """vda / dsa / kda / gmla layers: whole-sequence logits recorded from the reference classes, on the full-matrix
    routes (cases a, b, c at 1024 tokens) and beyond the 1024-key switch (case c at 1100 tokens, where KDA's
    chunk-wise route counts an anchor inside the window slice twice)."""
    from oracle import delta as OD
    g = golden("delta_reference.npz")
    for n in (1, 5, 6, 9, 10, 14):
        assert list(g[f"pattern_{n}"]) == OD.build_verse_delta_pattern(n)
    for tag in ("a", "b"):
        cfg, sd = OD.golden_case(tag)
        lg, _ = OM.forward(sd, cfg, g[tag + "_tokens"])
        np.testing.assert_allclose(lg, g[tag + "_logits"], rtol=2e-4, atol=2e-5)
    cfg, sd = OD.golden_case("c")
    rows = g["c_rows"]
    lg, _ = OM.forward(sd, cfg, g["c_tokens"])
    np.testing.assert_allclose(lg[:, rows], g["c_logits"], rtol=2e-4, atol=2e-5)
    lg, _ = OM.forward(sd, cfg, g["c_tokens"][:, :1024])
    np.testing.assert_allclose(lg[:, rows[:11]], g["c_logits_1024"], rtol=2e-4, atol=2e-5)
    # greedy continuation, token for token
    cfg, sd = OD.golden_case("a")
    cur = g["a_greedy"][:, :8]
    for _ in range(24):
        nxt = np.argmax(OM.forward(sd, cfg, cur)[0][:, -1], -1)
        cur = np.concatenate([cur, nxt[:, None]], axis=1)
    np.testing.assert_array_equal(cur, g["a_greedy"])


def test_delta_cache_and_tree_equal_the_whole_sequence_forward():
    from oracle import delta as OD
    cfg, sd = OD.golden_case("a")
    rng = np.random.default_rng(3)
    toks = rng.integers(0, cfg.vocab_size, (2, 30))
    full, _ = OM.forward(sd, cfg, toks)
    l1, cache = OM.forward(sd, cfg, toks[:, :17])
    l2, cache2 = OM.forward(sd, cfg, toks[:, 17:], cache=cache)
    np.testing.assert_allclose(np.concatenate([l1, l2], 1), full, rtol=2e-4, atol=2e-5)
    # commit keeps a prefix of the appended entries in every nested plane
    kept = OM.commit_cache(cache2, 17, [0, 1, 2])
    assert OM.cache_len(kept) == 20
    l3, _ = OM.forward(sd, cfg, toks[:, 20:], cache=kept)
    np.testing.assert_allclose(l3, full[:, 20:], rtol=2e-4, atol=2e-5)
    parents = [-1, -1, 0, 0, 1, 2, 2, 5]
    nodes = rng.integers(0, cfg.vocab_size, (1, len(parents)))
    _, cache = OM.forward(sd, cfg, toks[:1, :20])
    lg_tree, _ = OM.forward(sd, cfg, nodes, cache=cache, parents=parents)
    for i in range(len(parents)):
        path, j = [], i
        while j >= 0:
            path.append(j)
            j = parents[j]
        seq = np.concatenate([toks[:1, :20], nodes[:, path[::-1]]], axis=1)
        lg, _ = OM.forward(sd, cfg, seq)
        np.testing.assert_allclose(lg_tree[:, i], lg[:, -1], rtol=2e-4, atol=2e-5)


def test_delta_one_token_route_against_the_reference(golden):
    """`forward_recurrent` of the delta classes past 1024 keys (DSA stays dense, KDA keeps its plain mask, only GMLA
    switches to the window) and `generate` with its defaults on a delta model."""
    from oracle import delta as OD
    g = golden("delta_reference.npz")
    cfg, sd = OD.golden_case("c")
    got, _ = OM.forward(sd, cfg, g["c_tokens"][:, :1040], recurrent=True)
    np.testing.assert_allclose(got[:, g["c_recurrent_rows"]], g["c_recurrent_logits"], rtol=2e-4, atol=2e-5)
    cfg, sd = OD.golden_case("a")
    out = OM.generate_greedy_recurrent(sd, cfg, g["a_tokens"][:, :8], 24)
    np.testing.assert_array_equal(out, g["a_generate_default"])
