"""Layers of the delta attention kinds (vda / dsa / kda / gmla, verse_nex/delta_attention.py) on the device, against
logits recorded from the reference classes (tests/golden/delta_reference.npz) and against the CPU oracle."""

import numpy as np
import pytest

from oracle import delta as OD
from oracle import model as OM

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    return float(np.max(np.abs(np.asarray(a, np.float64) - b)) / max(np.max(np.abs(b)), 1e-30))


def build(cfg, sd, dtype="f32"):
    import versenext_b200 as vn
    kw = cfg.to_dict()
    kw.pop("init_std")
    m = vn.VerseNexLM(dtype=dtype, **kw)
    m.load_state_dict(sd)
    return m


@pytest.mark.parametrize("dtype,tol", [("f32", 1e-3), ("bf16", 2e-2)])
def test_delta_layers_against_the_reference_logits(golden, dtype, tol):
    """Whole-sequence logits: one layer of every kind with RoPE and GQA (a), no RoPE / multi-head / narrow latent
    (b), and the model of case c at 1024 keys (full-matrix routes) and at 1100 keys (window fall-backs; KDA counts an
    anchor inside its chunk's window slice twice)."""
    g = golden("delta_reference.npz")
    for tag in ("a", "b", "c"):
        cfg, sd = OD.golden_case(tag)
        if dtype == "bf16":        # the oracle run on the same bf16-rounded weights
            sd = {n: OM.bf16_round(v) for n, v in sd.items()}
        m = build(cfg, sd, dtype)
        toks = g[tag + "_tokens"]
        if tag != "c":
            ref = g[tag + "_logits"] if dtype == "f32" else OM.forward(sd, cfg, toks)[0]
            assert rel_err(m(toks).data.numpy(), ref) < tol, tag
            continue
        rows = g["c_rows"]
        for n, key, sel in ((1100, "c_logits", rows), (1024, "c_logits_1024", rows[:11])):
            ref = g[key] if dtype == "f32" else OM.forward(sd, cfg, toks[:, :n])[0][:, sel]
            assert rel_err(m(toks[:, :n]).data.numpy()[:, sel], ref) < tol, (tag, n)


def test_delta_cache_chain_tree_and_commit():
    """New positions on top of the cache equal the whole-sequence forward: a chain, a tree (every node against the
    forward over its own path), a committed path, and a chain that crosses the 1024-key switch."""
    cfg, sd = OD.golden_case("a")
    m = build(cfg, sd)
    rng = np.random.default_rng(3)
    toks = rng.integers(0, cfg.vocab_size, (2, 30))
    full = OM.forward(sd, cfg, toks)[0]
    cache = m.new_cache(2, 64)
    l1 = m.forward_cached(toks[:, :17], cache).numpy()
    cache.commit(17, np.full(2, 17, np.int32))
    l2 = m.forward_cached(toks[:, 17:], cache).numpy()
    assert rel_err(np.concatenate([l1, l2], 1), full) < 1e-3
    # keep 3 of the 13 appended entries, run the rest again
    cache.commit(13, np.full(2, 3, np.int32))
    np.testing.assert_array_equal(cache.per_seq_lens, [20, 20])
    l3 = m.forward_cached(toks[:, 20:], cache).numpy()
    assert rel_err(l3, full[:, 20:]) < 1e-3
    # tree on top of 20 cached tokens; then commit the path 1 -> 4 and continue
    parents = [-1, -1, 0, 0, 1, 2, 2, 5]
    nodes = rng.integers(0, cfg.vocab_size, (2, len(parents)))
    lt = m.forward_cached(nodes, cache, parents=parents).numpy()
    _, oc = OM.forward(sd, cfg, toks[:, :20])
    want, _ = OM.forward(sd, cfg, nodes, cache=oc, parents=parents)
    assert rel_err(lt, want) < 1e-3
    cache.commit(len(parents), np.full(2, 2, np.int32), keep_idx=np.tile(np.array([1, 4, 0, 0], np.int32), (2, 1)))
    np.testing.assert_array_equal(cache.per_seq_lens, [22, 22])
    tail = rng.integers(0, cfg.vocab_size, (2, 5))
    seq = np.concatenate([toks[:, :20], nodes[:, [1, 4]], tail], axis=1)
    l4 = m.forward_cached(tail, cache).numpy()
    assert rel_err(l4, OM.forward(sd, cfg, seq)[0][:, 22:]) < 1e-3
    m.check()
    # 1020 cached keys + 8 new ones: the new rows are beyond the switch, their keys are cached and new ones
    cfg, sd = OD.golden_case("c")
    m = build(cfg, sd)
    toks = rng.integers(0, cfg.vocab_size, (1, 1028))
    cache = m.new_cache(1, 1100)
    m.forward_cached(toks[:, :1020], cache, last_only=True)
    cache.commit(1020, np.full(1, 1020, np.int32))
    got = m.forward_cached(toks[:, 1020:], cache).numpy()
    _, oc = OM.forward(sd, cfg, toks[:, :1020])
    want, _ = OM.forward(sd, cfg, toks[:, 1020:], cache=oc)
    assert rel_err(got, want) < 1e-3
    m.check()


def test_delta_model_generates_and_verifies_like_the_reference(golden):
    """Greedy generation equals the stream recorded from the reference; the speculative engines (chain and tree) with
    a delta target commit exactly that stream, whatever the draft proposes."""
    import versenext_b200 as vn
    g = golden("delta_reference.npz")
    cfg, sd = OD.golden_case("a")
    t = build(cfg, sd)
    prompt = g["a_greedy"][:, :8]
    np.testing.assert_array_equal(t.generate(prompt, max_new_tokens=24, temperature=0.0), g["a_greedy"])
    d_cfg = OM.Config(vocab_size=cfg.vocab_size, dim=32, n_layer=2, n_head=2, n_kv_head=1, layer_pattern=["gmla", "kda"],
                      window_size=8, num_global_tokens=4, anchor_interval=4, use_alibi=False, use_rope=True,
                      max_seq_len=64, init_std=0.1)
    d = build(d_cfg, OM.init_state_dict(d_cfg, seed=41, gate_std=1.0))
    eng = vn.SpecEngine(t, d, max_batch=2, max_seq=64, k=3, temperature=0.0, bonus=True, max_new_tokens=32)
    toks, _ = eng.generate(prompt, 24)
    np.testing.assert_array_equal(toks[:, :32], g["a_greedy"])
    tree = vn.TreeSpecEngine(t, d, [-1, -1, 0, 0, 1, 2], max_batch=2, max_seq=64, max_new_tokens=32)
    toks, _ = tree.generate(prompt, 24)
    np.testing.assert_array_equal(toks[:, :32], g["a_greedy"])
    assert vn.build_verse_delta_pattern(10) == list(g["pattern_10"])


@pytest.mark.parametrize("n_kv", [2, 4, 1])
def test_delta_layers_bf16_head_dim_64_with_a_long_prompt(n_kv):
    """head_dim 64, bf16, 320 prompt rows (the projections then run as 256-row segments on the tcgen05 kernel) and a
    decode step on the cache; grouped-query (2 heads per KV head), multi-head and multi-query layouts."""
    cfg = OM.Config(vocab_size=128, dim=256, n_layer=2, n_head=4, n_kv_head=n_kv, layer_pattern=["vda", "dsa"],
                    window_size=32, num_global_tokens=8, anchor_interval=16, latent_dim=64, use_alibi=False,
                    use_rope=True, max_seq_len=256, init_std=0.05)
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=51, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    rng = np.random.default_rng(5)
    toks = rng.integers(0, cfg.vocab_size, (2, 161))
    want = OM.forward(sd, cfg, toks)[0]
    cache = m.new_cache(2, 256)
    l1 = m.forward_cached(toks[:, :160], cache).numpy()
    cache.commit(160, np.full(2, 160, np.int32))
    l2 = m.forward_cached(toks[:, 160:], cache).numpy()
    assert rel_err(l1, want[:, :160]) < 2e-2
    assert rel_err(l2, want[:, 160:]) < 2e-2
    m.check()


def hd64_delta_cfg(**over):
    kw = dict(vocab_size=128, dim=128, n_layer=4, n_head=2, n_kv_head=1, layer_pattern=["vda", "kda", "gmla", "dsa"],
              window_size=48, num_global_tokens=5, anchor_interval=40, latent_dim=32, use_alibi=False, use_rope=True,
              max_seq_len=2048, init_std=0.08)
    kw.update(over)
    return OM.Config(**kw)


def test_delta_tensor_core_routes_around_the_1024_key_switch():
    """bf16, head_dim 64: the modules run on the tensor-core attention kernel and (up to 256 rows) on the split-K
    tcgen05 GEMMs.  1100-token prompt (every class beyond its switch), a chain that crosses the switch on top of 1020
    cached keys, a tree whose nodes lie on both sides of it, and the same steps on the SIMT kernels
    (VN_ATTN_SIMT=1 at model creation) -- all against the oracle on the bf16-rounded weights."""
    import os
    cfg = hd64_delta_cfg()
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=61, gate_std=1.0).items()}
    rng = np.random.default_rng(7)
    toks = rng.integers(0, cfg.vocab_size, (1, 1100))
    # the oracle takes the prompt in the same pieces (a piece is on one side of the switch as a whole: the first four end
    # at or before 1024 keys, the last one beyond)
    want_pieces, oc = [], None
    for lo in range(0, 1100, 220):
        lg, oc = OM.forward(sd, cfg, toks[:, lo:lo + 220], cache=oc)
        want_pieces.append(lg)
    _, oc = OM.forward(sd, cfg, toks[:, :1020])
    want_chain = OM.forward(sd, cfg, toks[:, 1020:1030], cache=oc)[0]
    parents = [-1, -1, 0, 0, 1, 2, 2, 5, 7, 8]          # depths 0..5: positions 1020..1025, key counts 1021..1026
    nodes = rng.integers(0, cfg.vocab_size, (1, len(parents)))
    want_tree = OM.forward(sd, cfg, nodes, cache=oc, parents=parents)[0]
    for simt in ("0", "1"):
        os.environ["VN_ATTN_SIMT"] = simt
        try:
            m = build(cfg, sd, "bf16")
        finally:
            os.environ.pop("VN_ATTN_SIMT", None)
        cache = m.new_cache(1, 1200)
        for i, lo in enumerate(range(0, 1100, 220)):
            got = m.forward_cached(toks[:, lo:lo + 220], cache).numpy()
            cache.commit(220, np.full(1, 220, np.int32))
            assert rel_err(got, want_pieces[i]) < 2e-2, (simt, i)
        cache.reset()
        for lo in range(0, 1020, 255):
            m.forward_cached(toks[:, lo:lo + 255], cache, last_only=True)
            cache.commit(255, np.full(1, 255, np.int32))
        assert rel_err(m.forward_cached(toks[:, 1020:1030], cache).numpy(), want_chain) < 2e-2, simt
        assert rel_err(m.forward_cached(nodes, cache, parents=parents).numpy(), want_tree) < 2e-2, simt
        m.check()


def test_delta_and_trisparse_layers_in_one_model_bf16():
    """A model that mixes TriSparse, MoD and delta layers (the plane pairs of the cache are then not one per layer),
    batch 4: decode rows on the tcgen05 route against the oracle, and the engine's greedy stream against generate.
    The latent has the default width (n_kv_head * head_dim), so the GMLA module runs with its K | V projections folded
    through the latent into one matrix."""
    import versenext_b200 as vn
    # (every expert of a part is selected, top_k = E: the routed output is then continuous in the activations, and bf16
    # rounding cannot flip a choice between two experts with nearly equal router logits)
    cfg = hd64_delta_cfg(layer_pattern=["trisparse", "vda", "mod", "gmla"], num_dense_parts=2, num_experts_per_part=2,
                         top_k=2, window_size=16, anchor_interval=8, latent_dim=None)
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=71, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    rng = np.random.default_rng(9)
    toks = rng.integers(0, cfg.vocab_size, (4, 45))
    want = OM.forward(sd, cfg, toks)[0]
    cache = m.new_cache(4, 128)
    l1 = m.forward_cached(toks[:, :40], cache).numpy()
    cache.commit(40, np.full(4, 40, np.int32))
    l2 = m.forward_cached(toks[:, 40:], cache).numpy()
    assert rel_err(l1, want[:, :40]) < 2e-2
    assert rel_err(l2, want[:, 40:]) < 2e-2
    d_cfg = hd64_delta_cfg(n_layer=1, layer_pattern=["kda"])
    d = build(d_cfg, {n: OM.bf16_round(v) for n, v in OM.init_state_dict(d_cfg, seed=72, gate_std=1.0).items()}, "bf16")
    plain = m.generate(toks[:2, :12], max_new_tokens=20, temperature=0.0)
    spec = m.generate(toks[:2, :12], max_new_tokens=20, temperature=0.0, draft=d, k=3)
    np.testing.assert_array_equal(spec, plain)
    m.check()
    # a tensor loaded again after the first finalize: what finalize derives from it (the folded GMLA matrix) follows
    sd2 = dict(sd)
    name = "blocks.3.attn.w_k_up.weight"
    sd2[name] = OM.bf16_round(sd[name] * np.float32(-4.0))
    m.load_tensor(name, sd2[name])
    got = m(toks[:, :20]).data.numpy()
    assert rel_err(got, OM.forward(sd2, cfg, toks[:, :20])[0]) < 2e-2
    assert rel_err(got, want[:, :20]) > 4e-2            # and differs from what the old tensor gave


@pytest.mark.parametrize("dtype,tol", [("f32", 1e-3), ("bf16", 2e-2)])
def test_delta_one_token_route(golden, dtype, tol):
    """The reference's one-token route on a delta model: `forward_recurrent` token by token past 1024 keys against the
    recorded logits, `generate` with its defaults (greedy, last prompt token fed twice) against the recorded stream,
    and a prompt longer than 1024 tokens taken as one chunk on that route (every row then counts its own keys)."""
    g = golden("delta_reference.npz")
    cfg, sd = OD.golden_case("c")
    if dtype == "bf16":
        sd = {n: OM.bf16_round(v) for n, v in sd.items()}
    m = build(cfg, sd, dtype)
    toks = g["c_tokens"][:, :1040]
    rows = list(g["c_recurrent_rows"])
    want = g["c_recurrent_logits"] if dtype == "f32" else OM.forward(sd, cfg, toks, recurrent=True)[0][:, rows]
    states, got = None, []
    for t in range(1040):
        lg, states = m.forward_recurrent(toks[:, t:t + 1], states)
        if t in rows:
            got.append(lg.data.numpy()[:, 0])
    assert rel_err(np.stack(got, axis=1), want) < tol
    if dtype == "f32":
        out = m.generate(toks[:, :1030], max_new_tokens=6)
        np.testing.assert_array_equal(out, OM.generate_greedy_recurrent(sd, cfg, toks[:, :1030], 6))
        cfg, sd = OD.golden_case("a")
        m = build(cfg, sd)
        np.testing.assert_array_equal(m.generate(g["a_tokens"][:, :8], max_new_tokens=24), g["a_generate_default"])
    m.check()


def _dequantised(sd, scheme, names):
    """The state dict a model computes with after weight-only quantisation of `names` (oracle quantiser)."""
    from oracle import quant as OQ
    out = dict(sd)
    for n in names:
        w = sd[n]
        if scheme == "int8":
            out[n] = OQ.dequant_int8(*OQ.quantize_int8(w))
        elif scheme == "int4":
            out[n] = OQ.dequant_int4(*OQ.quantize_int4(w), w.shape[1])
        else:
            out[n] = OQ.dequant_int4_g128(*OQ.quantize_int4_g128(w), w.shape[1])
    return out


@pytest.mark.parametrize("scheme", ["int8", "int4", "int4g128"])
def test_delta_layers_weight_only_quantised(scheme):
    """The shipped mate preset is delta attention + INT4: every linear of the modules (stacked q|k|v, q|down, k|v up)
    is quantised like any other -- bytes and scales equal the oracle quantiser's, the forward equals the oracle on the
    dequantised weights (prompt rows and decode rows), and the same linears loaded in their quantised form give the
    same forward bit for bit."""
    from oracle import quant as OQ
    cfg = hd64_delta_cfg(latent_dim=64, window_size=16, anchor_interval=8)
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=81, gate_std=1.0).items()}
    names = [n for n, w in sd.items() if w.ndim == 2 and n.endswith(".weight") and "global_tokens" not in n
             and n != "tok_emb.weight"]
    m = build(cfg, sd, "bf16")
    m.quantize(scheme)
    for n in names + ["head.weight"]:
        w = sd["tok_emb.weight"] if n == "head.weight" else sd[n]
        q, s = m.read_quant(n)
        wq, ws = (OQ.quantize_int8(w) if scheme == "int8" else OQ.quantize_int4(w) if scheme == "int4"
                  else OQ.quantize_int4_g128(w))
        np.testing.assert_array_equal(q, wq, err_msg=n)
        np.testing.assert_array_equal(s.view(np.uint32), np.ascontiguousarray(ws).reshape(s.shape).view(np.uint32), err_msg=n)
    dq = _dequantised(sd, scheme, names)
    dq["head.weight"] = _dequantised({"h": sd["tok_emb.weight"]}, scheme, ["h"])["h"]
    o_cfg = OM.Config(**{**cfg.to_dict(), "tie_weights": False})
    rng = np.random.default_rng(11)
    toks = rng.integers(0, cfg.vocab_size, (2, 41))
    want = OM.forward(dq, o_cfg, toks)[0]
    cache = m.new_cache(2, 64)
    l1 = m.forward_cached(toks[:, :36], cache).numpy()
    cache.commit(36, np.full(2, 36, np.int32))
    l2 = m.forward_cached(toks[:, 36:], cache).numpy()
    assert rel_err(l1, want[:, :36]) < 3e-2
    assert rel_err(l2, want[:, 36:]) < 3e-2
    if scheme != "int4g128":
        class QL:                              # what a reference QuantizedLinear exposes (quantize.py:382-440)
            def __init__(self, w):
                self.qtype = scheme
                self.packed, self.scale = (OQ.quantize_int8 if scheme == "int8" else OQ.quantize_int4)(w)
        comp = {n: (QL(w) if n in names else w) for n, w in sd.items()}
        comp["head.weight"] = QL(sd["tok_emb.weight"])
        m2 = build(cfg, comp, "bf16")
        c2 = m2.new_cache(2, 64)
        np.testing.assert_array_equal(m2.forward_cached(toks[:, :36], c2).numpy(), l1)
        c2.commit(36, np.full(2, 36, np.int32))
        np.testing.assert_array_equal(m2.forward_cached(toks[:, 36:], c2).numpy(), l2)
    m.check()


def test_delta_one_token_route_on_the_tensor_core_kernels():
    """bf16, head_dim 64: the one-token route's rule (every row counts its own keys; no switch for DSA / KDA) on the
    tensor-core attention tile -- a 1030-token prompt taken as one chunk on that route, then single tokens."""
    cfg = hd64_delta_cfg()
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=91, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    rng = np.random.default_rng(13)
    toks = rng.integers(0, cfg.vocab_size, (1, 1040))
    want, oc = OM.forward(sd, cfg, toks[:, :1030], recurrent=True)
    cache = m.new_cache(1, 1100)
    m._set_recurrent(True)
    try:
        got = m.forward_cached(toks[:, :1030], cache).numpy()
        cache.commit(1030, np.full(1, 1030, np.int32))
        sel = [0, 1, 47, 48, 500, 1000, 1023, 1024, 1025, 1029]
        assert rel_err(got[:, sel], want[:, sel]) < 2e-2
        for t in range(1030, 1040):
            lg = m.forward_cached(toks[:, t:t + 1], cache).numpy()
            cache.commit(1, np.ones(1, np.int32))
            w, oc = OM.forward(sd, cfg, toks[:, t:t + 1], cache=oc, recurrent=True)
            assert rel_err(lg, w) < 2e-2, t
    finally:
        m._set_recurrent(False)
    # the whole-sequence rule gives something else beyond the switch (GMLA rows below 1024 keys differ)
    cache.reset()
    other = m.forward_cached(toks[:, :1030], cache).numpy()
    assert rel_err(other[:, [500]], want[:, [500]]) > 3e-2
    m.check()
