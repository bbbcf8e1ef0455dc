"""VerseNexLM forward, KV cache, tree verification and the speculative engine on the device,
against fixtures recorded from the reference and against the CPU oracle."""

import numpy as np
import pytest

from oracle import model as OM
from oracle import spec as OS

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    return float(np.max(np.abs(np.asarray(a, np.float64) - b)) / max(np.max(np.abs(b)), 1e-30))


def build(cfg: OM.Config, sd, dtype="f32"):
    import versenext_b200 as vn
    kw = cfg.to_dict()
    kw.pop("init_std")
    m = vn.VerseNexLM(dtype=dtype, **kw)
    m.load_state_dict(sd)
    return m


def _sd(g, prefix):
    return {n[len(prefix):]: g[n] for n in g.files if n.startswith(prefix)}


def variant_b():
    t_cfg = OM.small_config(tie_weights=False, init_std=0.2)
    d_cfg = OM.small_config(n_layer=1, tie_weights=False, init_std=0.2)
    t_sd = OM.init_state_dict(t_cfg, seed=101, gate_std=1.0)
    d_sd = OM.init_state_dict(d_cfg, seed=102, gate_std=1.0)
    d_sd["tok_emb.weight"], d_sd["head.weight"] = t_sd["tok_emb.weight"], t_sd["head.weight"]
    for n in list(d_sd):
        if n.startswith("blocks.0.") and not n.endswith("norm1.weight") and not n.endswith("norm2.weight"):
            d_sd[n] = (t_sd[n] + 0.15 * d_sd[n]).astype(np.float32)
    return t_cfg, t_sd, d_cfg, d_sd


def mini_cfg(**over):
    kw = dict(vocab_size=512, dim=64, n_layer=4, n_head=4, n_kv_head=2, window_size=16,
              num_global_tokens=8, max_seq_len=128, init_std=0.1)
    kw.update(over)
    return OM.mate_config(**kw)


def test_small_config_logits_and_greedy_stream(golden):
    """The small CPU-runnable configuration with the reference's own initial weights: logits 1e-3, greedy stream bit-exact."""
    g = golden("model_small.npz")
    cfg = OM.small_config()
    m = build(cfg, _sd(g, "a_t."))
    lg = m(g["prompt"]).data.numpy()
    assert rel_err(lg, g["a_logits"]) < 1e-3
    # temperature 0 takes the reference's whole-sequence route (arg-max of `forward`'s last row, cometspark.py:892-893)
    out = m.generate(g["prompt"], max_new_tokens=128, temperature=0.0)
    np.testing.assert_array_equal(out, g["a_greedy"])


def test_small_config_speculative_streams(golden):
    import versenext_b200 as vn
    g = golden("model_small.npz")
    t = build(OM.small_config(), _sd(g, "a_t."))
    d = build(OM.small_config(n_layer=1), _sd(g, "a_d."))
    eng = vn.SpecEngine(t, d, max_batch=1, max_seq=256, k=4, temperature=0.0, bonus=False, max_new_tokens=160)
    toks, st = eng.generate(g["prompt"], 128)
    np.testing.assert_array_equal(toks, g["a_spec"])
    assert st["rounds"] == int(g["a_rounds"])


def test_nondegenerate_variant_matches_reference_streams(golden):
    """Seeded weights with many rejections: logits, greedy stream, speculative stream, round and accept counts."""
    import versenext_b200 as vn
    g = golden("model_small.npz")
    t_cfg, t_sd, d_cfg, d_sd = variant_b()
    t, d = build(t_cfg, t_sd), build(d_cfg, d_sd)
    assert rel_err(t(g["prompt"]).data.numpy(), g["b_logits"]) < 1e-3
    np.testing.assert_array_equal(t.generate(g["prompt"], max_new_tokens=96, temperature=0.0), g["b_greedy"])
    eng = vn.SpecEngine(t, d, max_batch=1, max_seq=256, k=4, temperature=0.0, bonus=False, max_new_tokens=128)
    eng.prefill(g["prompt"])
    rounds = accepted = 0
    while int(eng.counts()[0]) < 96:
        eng.step()
        rounds += 1
        n = int(eng.accept_len.numpy()[0])
        accepted += n
    np.testing.assert_array_equal(eng.tokens(96), g["b_spec"][:, 32:])
    assert rounds == int(g["b_rounds"]) and accepted == int(g["b_accepted"])
    # with the bonus token the stream is still the greedy stream, in fewer rounds
    eng2 = vn.SpecEngine(t, d, max_batch=1, max_seq=256, k=4, temperature=0.0, bonus=True, max_new_tokens=128)
    toks, st = eng2.generate(g["prompt"], 96)
    np.testing.assert_array_equal(toks, g["b_greedy"])
    assert st["rounds"] <= rounds


@pytest.mark.parametrize("dtype,tol", [("f32", 1e-3), ("bf16", 2e-2)])
def test_mini_mate_model_against_reference(golden, dtype, tol):
    """MoD + TriSparse, RoPE, GQA, tied head, embedding scale; batch 2, beyond two windows."""
    g = golden("model_mini.npz")
    cfg = mini_cfg()
    sd = OM.init_state_dict(cfg, seed=7, gate_std=1.0)
    ref = g["logits"]
    if dtype == "bf16":  # the reference run with the same bf16-rounded weights
        sd = {n: OM.bf16_round(v) for n, v in sd.items()}
        ref = OM.forward(sd, cfg, g["tokens"])[0]
    m = build(cfg, sd, dtype)
    lg = m(g["tokens"]).data.numpy()
    assert rel_err(lg, ref) < tol
    if dtype == "f32":
        m2 = build(mini_cfg(embedding_scale=False, use_alibi=True), sd)
        assert rel_err(m2(g["tokens"][:1]).data.numpy(), g["logits_alibi_rope"]) < tol
    # cached continuation: prefill 30 then 10 more positions
    cache = m.new_cache(2, 64)
    m.forward_cached(g["tokens"][:, :30], cache, want_logits=False, want_hidden=True, last_only=True)
    cache.commit(30, np.full(2, 30, np.int32))
    np.testing.assert_array_equal(cache.per_seq_lens, [30, 30])
    lg2 = m.forward_cached(g["tokens"][:, 30:], cache).numpy()
    want = g["logits_incremental"] if dtype == "f32" else ref[:, 30:]
    assert rel_err(lg2, want) < tol


def test_ragged_batch_lengths_and_reset():
    cfg = mini_cfg(n_layer=2)
    sd = OM.init_state_dict(cfg, seed=3, gate_std=0.5)
    m = build(cfg, sd)
    rng = np.random.default_rng(1)
    a, b = rng.integers(0, 512, (1, 21)), rng.integers(0, 512, (1, 9))
    cache = m.new_cache(2, 64)
    # sequence 0 holds 21 tokens, sequence 1 holds 9: feed them separately via set_lengths
    both = np.concatenate([a[:, :9], b], axis=0)
    m.forward_cached(both, cache, want_logits=False, want_hidden=True, last_only=True)
    cache.commit(9, np.array([9, 9], np.int32))
    pad = np.concatenate([a[:, 9:], np.zeros((1, 12), np.int64)], axis=0)
    m.forward_cached(pad, cache, want_logits=False, want_hidden=True, last_only=True)
    cache.commit(12, np.array([12, 0], np.int32))          # sequence 1 rolls back all 12
    np.testing.assert_array_equal(cache.per_seq_lens, [21, 9])
    nxt = rng.integers(0, 512, (2, 3))
    lg = m.forward_cached(nxt, cache).numpy()
    wa = OM.forward(sd, cfg, np.concatenate([a, nxt[:1]], axis=1))[0][:, -3:]
    wb = OM.forward(sd, cfg, np.concatenate([b, nxt[1:]], axis=1))[0][:, -3:]
    assert rel_err(lg[0], wa[0]) < 1e-3 and rel_err(lg[1], wb[0]) < 1e-3
    cache.reset_seq(1)
    np.testing.assert_array_equal(cache.per_seq_lens, [21, 0])
    k0, v0 = cache.get(0, 0)
    _, oc = OM.forward(sd, cfg, a)
    np.testing.assert_allclose(k0, oc[0]["k"][0], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(v0, oc[0]["v"][0], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype,tol", [("f32", 1e-3), ("bf16", 2e-2)])
def test_tree_verification_equals_per_path_forward(dtype, tol):
    """16-node tree (4 roots, 2 children under the first two, 2 grandchildren under each child)."""
    cfg = mini_cfg(n_layer=3, window_size=12)
    sd = OM.init_state_dict(cfg, seed=9, gate_std=1.0)
    if dtype == "bf16":
        sd = {n: OM.bf16_round(v) for n, v in sd.items()}
    m = build(cfg, sd, dtype)
    rng = np.random.default_rng(2)
    B = 2
    ctx_tok = rng.integers(0, 512, (B, 20))
    parents = [-1, -1, -1, -1, 0, 0, 1, 1, 4, 4, 5, 5, 6, 6, 7, 7]
    nodes = rng.integers(0, 512, (B, 16))
    cache = m.new_cache(B, 64)
    m.forward_cached(ctx_tok, cache, want_logits=False, want_hidden=True, last_only=True)
    cache.commit(20, np.full(B, 20, np.int32))
    lg = m.forward_cached(nodes, cache, parents=parents).numpy()
    _, oc = OM.forward(sd, cfg, ctx_tok)
    want, _ = OM.forward(sd, cfg, nodes, cache=oc, parents=parents)
    assert rel_err(lg, want) < tol
    # commit the path 1 -> 6 -> 13 of sequence 0 and 0 -> 5 of sequence 1, then continue
    keep = np.array([[1, 6, 13], [0, 5, 0]], np.int32)
    cache.commit(16, np.array([3, 2], np.int32), keep_idx=keep)
    np.testing.assert_array_equal(cache.per_seq_lens, [23, 22])
    nxt = rng.integers(0, 512, (B, 2))
    lg2 = m.forward_cached(nxt, cache).numpy()
    s0 = np.concatenate([ctx_tok[:1], nodes[:1, [1, 6, 13]], nxt[:1]], axis=1)
    s1 = np.concatenate([ctx_tok[1:], nodes[1:, [0, 5]], nxt[1:]], axis=1)
    assert rel_err(lg2[0], OM.forward(sd, cfg, s0)[0][0, -2:]) < tol
    assert rel_err(lg2[1], OM.forward(sd, cfg, s1)[0][0, -2:]) < tol


def test_batched_stochastic_engine_matches_oracle():
    """temperature 0.8, top-k 20, batch 3: tokens identical to the CPU restatement with the same Philox streams."""
    import versenext_b200 as vn
    t_cfg, t_sd, d_cfg, d_sd = variant_b()
    t, d = build(t_cfg, t_sd), build(d_cfg, d_sd)
    prompts = np.random.default_rng(5).integers(0, 256, (3, 12)).astype(np.int64)
    eng = vn.SpecEngine(t, d, max_batch=3, max_seq=128, k=3, temperature=0.8, top_k=20, seed=77, bonus=True,
                        max_new_tokens=64)
    toks, st = eng.generate(prompts, 24)
    want = OS.generate(t_sd, t_cfg, d_sd, d_cfg, prompts, 3, 24, temperature=0.8, top_k=20, seed=77, bonus=True)
    np.testing.assert_array_equal(toks, want["tokens"])


def test_forward_recurrent_matches_whole_sequence_forward():
    """CometSparkNexLM.forward_recurrent (cometspark.py:737-767): token by token with the returned states the
    logits equal those of one forward over the whole sequence; T != 1 is an AssertionError
    (tri_sparse_attn.py:635) and a full cache a RuntimeError."""
    cfg = OM.small_config()
    sd = OM.init_state_dict(cfg, seed=6)
    m = build(cfg, sd)
    toks = np.random.default_rng(6).integers(0, cfg.vocab_size, (2, 9))
    full = np.asarray(m(toks).data)
    states = None
    for t in range(toks.shape[1]):
        lg, states = m.forward_recurrent(toks[:, t:t + 1], states)
        assert lg.shape == (2, 1, cfg.vocab_size) and len(states) == cfg.n_layer
        assert rel_err(np.asarray(lg.data)[:, 0], full[:, t]) < 1e-3
    with pytest.raises(AssertionError):
        m.forward_recurrent(toks[:, :2], states)
    tiny = build(OM.small_config(max_seq_len=4), sd)
    st = None
    with pytest.raises(RuntimeError):
        for t in range(6):
            _, st = tiny.forward_recurrent(toks[:, t:t + 1], st)


def _recurrent_case(g, tag):
    cfg = (OM.small_config(tie_weights=False, init_std=0.2) if tag == "alibi" else
           OM.mate_config(vocab_size=512, dim=64, n_layer=2, n_head=4, n_kv_head=2, window_size=16,
                          num_global_tokens=8, max_seq_len=256, init_std=0.2, num_dense_parts=2,
                          num_experts_per_part=2, top_k=1, layer_pattern=["trisparse", "trisparse"],
                          embedding_scale=False))
    sd = {n[len(tag) + 1:]: g[n] for n in g.files if n.startswith(tag + ".")}
    return cfg, sd


@pytest.mark.parametrize("tag", ["alibi", "rope"])
def test_recurrent_route_against_the_reference_beyond_the_window(golden, tag):
    """`forward_recurrent` token by token for more than two windows, and `generate` with its default arguments
    (greedy on the recurrent route: last prompt token fed twice, EOS stop, EOS column appended) against what
    the reference's own methods returned for the same weights (tests/golden/recurrent_reference.npz)."""
    g = golden("recurrent_reference.npz")
    cfg, sd = _recurrent_case(g, tag)
    m = build(cfg, sd)
    toks, want = g[f"{tag}_tokens"], g[f"{tag}_recurrent_logits"]
    states = None
    got = []
    for t in range(toks.shape[1]):
        lg, states = m.forward_recurrent(toks[:, t:t + 1], states)
        got.append(np.asarray(lg.data)[:, 0])
    assert rel_err(np.stack(got, 1), want) < 1e-3
    W = cfg.window_size
    np.testing.assert_array_equal(m.generate(toks[:, :W + 5], max_new_tokens=W + 7), g[f"{tag}_generate"])
    eos = int(g[f"{tag}_generate"][0, W + 6])
    np.testing.assert_array_equal(m.generate(toks[:1, :6], max_new_tokens=12, eos_id=eos), g[f"{tag}_generate_eos"])


def test_generate_api_sampling_and_eos():
    cfg = OM.small_config()
    sd = OM.init_state_dict(cfg, seed=4)
    m = build(cfg, sd)
    p = np.array([[1, 2, 3, 4]], np.int64)
    out = m.generate(p, max_new_tokens=5, temperature=0.9, top_k=10, seed=3)
    assert out.shape == (1, 9) and out.dtype == np.int64 and np.all((out >= 0) & (out < 256))
    np.testing.assert_array_equal(out, m.generate(p, max_new_tokens=5, temperature=0.9, top_k=10, seed=3))
    out = m.generate(p[0], max_new_tokens=3, eos_id=255)
    assert out.shape[0] == 1 and out[0, -1] == 255


def test_errors():
    import versenext_b200 as vn
    with pytest.raises(ValueError):
        vn.VerseNexLM(vocab_size=16, dim=16, n_layer=2, n_head=2, layer_pattern=["trisparse"])
    with pytest.raises(ValueError):
        vn.VerseNexLM(vocab_size=16, dim=16, n_layer=1, n_head=2, layer_pattern=["rwkv"])
    cfg = OM.small_config()
    sd = OM.init_state_dict(cfg, seed=4)
    m = build(cfg, sd)
    cache = m.new_cache(1, 8)
    with pytest.raises(RuntimeError):
        m.forward_cached(np.zeros((1, 9), np.int64), cache)           # capacity
    with pytest.raises(IndexError):
        cache.get(7, 0, 1)
    with pytest.raises(IndexError):
        cache.reset_seq(3)
    with pytest.raises(ValueError):
        m.forward_cached(np.zeros((2, 2), np.int64), cache)           # batch larger than the cache
    with pytest.raises(IndexError):                                   # token id outside the vocabulary
        m(np.array([[1, 2, 10 ** 6]], np.int64))
    m.check()                                                         # the flag was cleared by the raise
    m2 = vn.VerseNexLM(vocab_size=16, dim=16, n_layer=1, n_head=2)
    with pytest.raises(ValueError):
        m2.finalize()                                                 # tensors missing
    with pytest.raises(ValueError):
        m2.load_tensor("blocks.0.attn.wq.weight", np.zeros((3, 3), np.float32))


def hd64_cfg(**over):
    kw = dict(vocab_size=384, dim=256, n_layer=2, n_head=4, n_kv_head=2, window_size=24, num_global_tokens=20,
              max_seq_len=256, init_std=0.05, num_dense_parts=2, num_experts_per_part=2, top_k=1)
    kw.update(over)
    return OM.mate_config(**kw)


@pytest.mark.parametrize("variant", ["rope_window", "alibi_norope", "tree"])
def test_tensor_core_attention_head_dim_64(variant):
    """bf16, head_dim 64 takes the tensor-core attention kernel: window edge, sinks, ALiBi path, GQA, trees."""
    over = {}
    if variant == "alibi_norope":
        over = dict(use_alibi=True, use_rope=False, embedding_scale=False)
    cfg = hd64_cfg(**over)
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=21, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    rng = np.random.default_rng(6)
    B = 3
    ctx_tok = rng.integers(0, 384, (B, 61))          # > 2 windows, not a multiple of 16
    cache = m.new_cache(B, 128)
    lg0 = m.forward_cached(ctx_tok, cache).numpy()   # prefill through the same kernel (many row tiles)
    want0, oc = OM.forward(sd, cfg, ctx_tok)
    assert rel_err(lg0, want0) < 2e-2
    cache.commit(61, np.full(B, 61, np.int32))
    if variant == "tree":
        parents = [-1, -1, -1, -1, 0, 0, 1, 1, 4, 4, 5, 5, 6, 6, 7, 7]
        nodes = rng.integers(0, 384, (B, 16))
        lg = m.forward_cached(nodes, cache, parents=parents).numpy()
        want, _ = OM.forward(sd, cfg, nodes, cache=oc, parents=parents)
    else:
        nxt = rng.integers(0, 384, (B, 5))
        lg = m.forward_cached(nxt, cache).numpy()
        want, _ = OM.forward(sd, cfg, nxt, cache=oc)
    assert rel_err(lg, want) < 2e-2


def test_fused_layer_stack_of_a_draft_model():
    """A small all-TriSparse bf16 model runs its layer stack as one cooperative kernel (bounded grid barriers between
    the phases).  Against the oracle and against the chain of separate kernels: decode steps of 1 and of 3 rows per
    sequence, GQA, window edge, sinks, ALiBi, ragged lengths; the launch count shows which route ran."""
    cfg = OM.small_config(vocab_size=384, dim=256, n_layer=3, n_head=4, n_kv_head=2, window_size=24,
                          num_global_tokens=20, max_seq_len=256)
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=33, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    ctx = m.ctx
    rng = np.random.default_rng(12)
    B = 5
    ctx_tok = rng.integers(0, 384, (B, 41))
    outs = {}
    for fused in (True, False):
        m.set_fused_stack(fused)
        cache = m.new_cache(B, 128)
        lg0 = m.forward_cached(ctx_tok, cache).numpy()          # 205 rows: the chain either way
        want0, oc = OM.forward(sd, cfg, ctx_tok)
        assert rel_err(lg0, want0) < 2e-2
        lens = np.array([41, 33, 17, 41, 2], np.int32)           # ragged: rows keep different prefixes
        cache.commit(41, lens)
        got = []
        for tn in (1, 3, 1):
            nxt = rng.integers(0, 384, (B, tn)) if fused else outs["tok"][len(got)]
            l0 = ctx.launch_count()
            lg = m.forward_cached(nxt, cache).numpy()
            n_launch = ctx.launch_count() - l0
            assert (n_launch <= 3) == fused, n_launch             # stack + head (+ nothing else) vs some twenty
            got.append((nxt, lg))
            cache.commit(tn, np.full(B, tn, np.int32))
        outs[fused] = got
        if fused:
            outs["tok"] = [g[0] for g in got]
    for (t1, a), (t2, b) in zip(outs[True], outs[False]):
        assert np.array_equal(t1, t2)
        assert rel_err(a, b) < 1e-2
    # last_only and the hidden rows
    m.set_fused_stack(True)
    cache = m.new_cache(B, 128)
    m.forward_cached(ctx_tok, cache, want_logits=False)
    cache.commit(41, np.full(B, 41, np.int32))
    nxt = rng.integers(0, 384, (B, 2))
    lg_last = m.forward_cached(nxt, cache, last_only=True).numpy()
    lg_all = m.forward_cached(nxt, cache).numpy()
    assert np.array_equal(lg_last.reshape(B, -1), lg_all[:, -1].reshape(B, -1))
    want, _ = OM.forward(sd, cfg, np.concatenate([ctx_tok, nxt], 1))
    assert rel_err(lg_all, want[:, -2:]) < 2e-2
    # a grid-barrier wait that runs out: one cycle is never enough for the CTAs to meet.  The kernel walks on and
    # terminates, the status turns into RuntimeError, and the next forward (barrier words reset) is right again.
    lib = ctx.lib
    ctx._check(lib.vn_model_set_wait_limit(m.handle, 1))
    try:
        m.forward_cached(nxt, cache, want_logits=False, want_hidden=True)     # the stack kernel alone, no GEMM
        with pytest.raises(RuntimeError):
            m.check()
    finally:
        ctx._check(lib.vn_model_set_wait_limit(m.handle, 0))
    m.check()
    assert np.array_equal(m.forward_cached(nxt, cache).numpy(), lg_all)


def test_prompt_gemms_on_the_tensor_core_kernel_in_row_segments(monkeypatch):
    """More than 256 rows (a prompt): the dense projections run on the tcgen05 kernel as segments of 256 rows that
    share one weight matrix.  393 rows = one full segment + 137 (no multiple of 16); against the oracle and against
    the mma.sync kernels; then a decode step on the cache the prompt left."""
    cfg = hd64_cfg()
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=41, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    rng = np.random.default_rng(14)
    B, T = 3, 131
    toks = rng.integers(0, 384, (B, T))
    want, oc = OM.forward(sd, cfg, toks)
    outs = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("VN_PREFILL_TC", flag)
        cache = m.new_cache(B, 192)
        l0 = m.ctx.launch_count()
        outs[flag] = m.forward_cached(toks, cache).numpy()
        assert rel_err(outs[flag], want) < 2e-2
        cache.commit(T, np.full(B, T, np.int32))
        nxt = rng.integers(0, 384, (B, 2)) if flag == "1" else nxt
        lg = m.forward_cached(nxt, cache).numpy()
        want2, _ = OM.forward(sd, cfg, nxt, cache=oc)
        assert rel_err(lg, want2) < 2e-2
    assert rel_err(outs["1"], outs["0"]) < 1e-2
    m.check()


@pytest.mark.parametrize("n_kv", [1, 2, 4])
def test_prompt_attention_kernel_shares_key_blocks_between_tiles(n_kv, monkeypatch):
    """Prompts of a RoPE model without ALiBi take the attention kernel whose eight warps hold eight row tiles and
    share the key blocks: a first chunk on an empty cache (window 24 shorter than the chunk, 20 sinks, 77 positions:
    no multiple of 16), a second chunk on top of it, ragged committed lengths; against the oracle and against the
    one-tile-per-CTA kernel; GQA with 4, 2 and 1 query heads per kv head."""
    cfg = hd64_cfg(n_kv_head=n_kv)
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=50 + n_kv, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    rng = np.random.default_rng(n_kv)
    B = 3
    c1, c2 = rng.integers(0, 384, (B, 77)), rng.integers(0, 384, (B, 45))
    want1, oc = OM.forward(sd, cfg, c1)
    want2, _ = OM.forward(sd, cfg, c2, cache=oc)
    got = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("VN_ATTN_PREFILL", flag)
        cache = m.new_cache(B, 160)
        a = m.forward_cached(c1, cache).numpy()
        cache.commit(77, np.full(B, 77, np.int32))
        b = m.forward_cached(c2, cache).numpy()
        assert rel_err(a, want1) < 2e-2 and rel_err(b, want2) < 2e-2
        got[flag] = (a, b)
        # ragged: sequences keep 77, 40 and 9 positions of the first chunk, then the second chunk again
        cache.set_lengths(np.array([77, 40, 9], np.int32))
        r = m.forward_cached(c2, cache).numpy()
        for i, keep in enumerate((77, 40, 9)):
            _, oci = OM.forward(sd, cfg, c1[i:i + 1, :keep])
            wi, _ = OM.forward(sd, cfg, c2[i:i + 1], cache=oci)
            assert rel_err(r[i:i + 1], wi) < 2e-2
    assert rel_err(got["1"][0], got["0"][0]) < 1e-2 and rel_err(got["1"][1], got["0"][1]) < 1e-2
    m.check()


def test_persistent_gemm_variant(monkeypatch):
    """Opt-in persistent tile-loop GEMM (one CTA per SM, double-buffered TMEM accumulator), forced onto the small
    shapes of this model: dense store, split-K partial and per-expert SwiGLU tiles give the same logits."""
    monkeypatch.setenv("VN_TC_PERSIST", "2")       # read at every GEMM launch
    cfg = hd64_cfg()
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=27, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    rng = np.random.default_rng(10)
    B = 4
    ctx_tok = rng.integers(0, 384, (B, 37))
    cache = m.new_cache(B, 128)
    lg0 = m.forward_cached(ctx_tok, cache).numpy()
    want0, oc = OM.forward(sd, cfg, ctx_tok)
    assert rel_err(lg0, want0) < 2e-2
    cache.commit(37, np.full(B, 37, np.int32))
    for _ in range(2):
        nxt = rng.integers(0, 384, (B, 5))
        lg = m.forward_cached(nxt, cache).numpy()
        want, oc = OM.forward(sd, cfg, nxt, cache=oc)
        assert rel_err(lg, want) < 2e-2
        cache.commit(5, np.full(B, 5, np.int32))


def _dequantise(w, scheme):
    from oracle import quant as OQ
    if scheme == "int8":
        q, s = OQ.quantize_int8(w)
        return OQ.dequant_int8(q, s)
    if scheme == "int4":
        p, s = OQ.quantize_int4(w)
        return OQ.dequant_int4(p, s, w.shape[1])
    p, s = OQ.quantize_int4_g128(w)
    return OQ.dequant_int4_g128(p, s, w.shape[1])


def _dequantised_state_dict(sd, cfg, scheme):
    """What the quantised device model computes with, as float32 weights for the oracle."""
    out = {}
    for n, w in sd.items():
        linear = w.ndim == 2 and n.endswith(".weight") and "global_tokens" not in n and "router" not in n \
            and n != "tok_emb.weight"
        out[n] = _dequantise(w, scheme) if linear else w
    if cfg.tie_weights:   # the head is quantised on its own copy, the embedding stays dense
        out["head.weight"] = _dequantise(sd["tok_emb.weight"], scheme)
    return out


@pytest.mark.parametrize("gemm", ["tcgen05", "mma"])
@pytest.mark.parametrize("scheme", ["int8", "int4", "int4g128"])
def test_weight_only_quantised_model(scheme, gemm, monkeypatch):
    """INT8 / INT4 per output channel (reference schemes) and INT4 group-128: the device model against the
    reference forward run on the dequantised weights; MoD + TriSparse, chain then cached continuation.  Both
    GEMM paths: raw bytes dequantised into the tcgen05 operand stage (default), and the mma.sync kernels."""
    monkeypatch.setenv("VN_GEMM_TCQ", "1" if gemm == "tcgen05" else "0")     # read when the model is quantised
    cfg = OM.mate_config(vocab_size=320, dim=128, n_layer=2, n_head=4, n_kv_head=2, window_size=16,
                         num_global_tokens=8, max_seq_len=128, init_std=0.08, num_dense_parts=2,
                         num_experts_per_part=2, top_k=1, expert_hidden=192, mlp_hidden_multiple=3)
    assert cfg.mlp_hidden % 128 == 0 and cfg.expert_hidden % 128 == 64    # expert w_down: a half last group
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=31, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    m.quantize(scheme)
    sd_q = _dequantised_state_dict(sd, cfg, scheme)
    oracle_cfg = OM.Config(**{**cfg.to_dict(), "tie_weights": False})
    toks = np.random.default_rng(8).integers(0, 320, (2, 30))
    cache = m.new_cache(2, 64)
    lg = m.forward_cached(toks[:, :24], cache).numpy()
    want, oc = OM.forward(sd_q, oracle_cfg, toks[:, :24])
    assert rel_err(lg, want) < 2e-2
    cache.commit(24, np.full(2, 24, np.int32))
    lg2 = m.forward_cached(toks[:, 24:], cache).numpy()
    want2, _ = OM.forward(sd_q, oracle_cfg, toks[:, 24:], cache=oc)
    assert rel_err(lg2, want2) < 2e-2
    with pytest.raises(ValueError):
        m.load_tensor("norm.weight", np.ones(128, np.float32))
    with pytest.raises(ValueError):
        m.quantize("int8")


@pytest.mark.parametrize("scheme,tol", [("int8", 2e-3), ("int4", 2e-3), ("int4g128", 1e-2)])
def test_quantised_tcgen05_gemm_equals_mma_gemm(scheme, tol, monkeypatch):
    """185 rows (six 32-token accumulator chunks over both epilogue groups, a ragged last one), head_dim 64,
    routed experts with uneven segment sizes: the tcgen05 path must reproduce the mma.sync path, which applies
    the scales to fp32 accumulators.  Per-row schemes feed identical integer operands to both (only the fp32
    summation order differs); group-128 rounds q * scale to bf16 in the operand (relative 2^-9 per weight)."""
    cfg = hd64_cfg()
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=29, gate_std=1.0).items()}
    rng = np.random.default_rng(12)
    B = 5
    ctx_tok = rng.integers(0, 384, (B, 37))
    nxt = rng.integers(0, 384, (B, 5))
    outs = []
    for flag in ("0", "1"):
        monkeypatch.setenv("VN_GEMM_TCQ", flag)
        m = build(cfg, sd, "bf16")
        m.quantize(scheme)
        cache = m.new_cache(B, 128)
        a = m.forward_cached(ctx_tok, cache).numpy()
        cache.commit(37, np.full(B, 37, np.int32))
        b = m.forward_cached(nxt, cache).numpy()
        m.check()
        outs.append((a, b))
    assert np.isfinite(outs[1][0]).all() and np.isfinite(outs[1][1]).all()
    assert rel_err(outs[1][0], outs[0][0]) < tol
    assert rel_err(outs[1][1], outs[0][1]) < tol


@pytest.mark.parametrize("scheme", ["int8", "int4g128"])
def test_quantised_head_on_a_column_range(scheme):
    """A rank that owns vocabulary columns [lo, hi) of a quantised target: its slice of the head (raw bytes and
    scales offset by whole rows) gives the same logits as those columns of the full quantised forward."""
    cfg = hd64_cfg()
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=30, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    m.quantize(scheme)
    toks = np.random.default_rng(13).integers(0, 384, (3, 9))
    cache = m.new_cache(3, 32)
    lg, hid = m.forward_cached(toks, cache, want_hidden=True)
    full = lg.numpy().reshape(27, 384)
    for lo, hi in ((0, 128), (128, 384), (256, 384)):
        part = m.head_columns(hid, lo, hi - lo).numpy()
        np.testing.assert_allclose(part, full[:, lo:hi], rtol=0, atol=1e-5)
    m.check()


def test_quantise_needs_bf16_and_known_scheme():
    cfg = OM.small_config()
    m = build(cfg, OM.init_state_dict(cfg, seed=4))
    with pytest.raises(NotImplementedError):
        m.quantize("int8")
    with pytest.raises(ValueError):
        m.quantize("fp3")


# ---- generate() and serving through the speculative engine ---------------------------------------------------------
def test_generate_through_the_engine_equals_the_reference_streams(golden):
    """`generate(..., draft=...)`: greedy decoding routed through the speculative engine gives the reference's
    greedy streams (whole-sequence route, temperature 0) and the recurrent route's output (default arguments:
    last prompt token fed twice) token for token."""
    g = golden("model_small.npz")
    t = build(OM.small_config(), _sd(g, "a_t."))
    d = build(OM.small_config(n_layer=1), _sd(g, "a_d."))
    np.testing.assert_array_equal(t.generate(g["prompt"], max_new_tokens=128, temperature=0.0, draft=d), g["a_greedy"])
    t_cfg, t_sd, d_cfg, d_sd = variant_b()
    t2, d2 = build(t_cfg, t_sd), build(d_cfg, d_sd)
    np.testing.assert_array_equal(t2.generate(g["prompt"], max_new_tokens=96, temperature=0.0, draft=d2, k=3), g["b_greedy"])
    r = golden("recurrent_reference.npz")
    for tag in ("alibi", "rope"):
        cfg, sd = _recurrent_case(r, tag)
        m = build(cfg, sd)
        dsd = dict(sd)
        toks = r[f"{tag}_tokens"]
        W = cfg.window_size
        # the model drafts for itself: every proposal is accepted, the stream is the reference's
        np.testing.assert_array_equal(m.generate(toks[:, :W + 5], max_new_tokens=W + 7, draft=m), r[f"{tag}_generate"])
        eos = int(r[f"{tag}_generate"][0, W + 6])
        np.testing.assert_array_equal(m.generate(toks[:1, :6], max_new_tokens=12, eos_id=eos, draft=m),
                                      r[f"{tag}_generate_eos"])


CFG3_TREE = [-1, -1, -1, -1, 0, 0, 1, 1, 4, 4, 5, 5, 6, 6, 7, 7]


def test_top_m_and_greedy_tree_acceptance_kernels():
    """`vn_top_m` against a stable sort (ties to the lower id), `vn_tree_accept_greedy` against a walk in Python on
    random trees' tokens: accepted path, committed tokens, the slot lists for both caches."""
    import ctypes as C
    import versenext_b200 as vn
    ctx = vn.Context.get(0)
    lib = ctx.lib
    rng = np.random.default_rng(8)
    R, V = 5, 3001
    x = rng.integers(-6, 6, (R, V)).astype(np.float32)             # many ties
    xd = ctx.from_numpy(x)
    for m in (1, 3, 8):
        out = ctx.zeros((R, 9), np.int64)
        ctx._check(lib.vn_top_m(ctx.handle, C.c_void_p(xd.ptr), V, R, V, m, C.c_void_p(out.ptr), 9))
        want = np.argsort(-x, axis=-1, kind="stable")[:, :m]
        np.testing.assert_array_equal(out.numpy()[:, :m], want)
    with pytest.raises(ValueError):
        ctx._check(lib.vn_top_m(ctx.handle, C.c_void_p(xd.ptr), V, R, V, 9, C.c_void_p(out.ptr), 9))
    parents, B, D = CFG3_TREE, 64, 3
    T = len(parents) + 1
    prow = np.array([-1] + [p + 1 for p in parents], np.int32)
    tok = rng.integers(0, 6, (B, T)).astype(np.int64)
    arg = rng.integers(0, 6, (B, T)).astype(np.int64)
    for b in range(0, B, 3):                                        # make long paths likely in a third of the rows
        cur = 0
        for _ in range(D):
            kids = [c for c in range(T) if prow[c] == cur]
            if not kids:
                break
            nxt = kids[rng.integers(0, len(kids))]
            arg[b, cur] = tok[b, nxt]
            cur = nxt
    o_len, o_tok = ctx.zeros((B,), np.int32), ctx.zeros((B, D + 1), np.int64)
    kt, kd = ctx.zeros((B, D + 1), np.int32), ctx.zeros((B, D + 1), np.int32)
    tok_d, arg_d, prow_d = ctx.from_numpy(tok), ctx.from_numpy(arg), ctx.from_numpy(prow)     # kept alive over the call
    ctx._check(lib.vn_tree_accept_greedy(ctx.handle, C.c_void_p(tok_d.ptr), C.c_void_p(arg_d.ptr),
                                         C.c_void_p(prow_d.ptr), B, T, D, C.c_void_p(o_len.ptr),
                                         C.c_void_p(o_tok.ptr), C.c_void_p(kt.ptr), C.c_void_p(kd.ptr)))
    o_len, o_tok, kt, kd = o_len.numpy(), o_tok.numpy(), kt.numpy(), kd.numpy()
    seen = set()
    for b in range(B):
        cur, path = 0, []
        while len(path) < D:
            hit = [c for c in range(cur + 1, T) if prow[c] == cur and tok[b, c] == arg[b, cur]]
            if not hit:
                break
            path.append(hit[0])
            cur = hit[0]
        a = len(path)
        seen.add(a)
        assert o_len[b] == a
        want_tok = [tok[b, r] for r in path] + [arg[b, cur]] + [-1] * (D - a)
        np.testing.assert_array_equal(o_tok[b], want_tok)
        np.testing.assert_array_equal(kt[b, :a + 1], [0] + path)
        np.testing.assert_array_equal(kd[b, :a + 1], ([0, 1] + [r + 1 for r in path])[:a + 1])
    assert {0, 1, 2, 3} <= seen


def test_tree_engine_commits_the_targets_greedy_stream(golden):
    """Tree proposals (configuration 3's 16-node tree, and a plain chain written as a tree): the committed tokens are
    the reference's greedy streams token for token, with a draft that often agrees (variant b) and one that rarely
    does; more than one token per round is committed where the draft agrees."""
    import versenext_b200 as vn
    g = golden("model_small.npz")
    t = build(OM.small_config(), _sd(g, "a_t."))
    d = build(OM.small_config(n_layer=1), _sd(g, "a_d."))
    eng = vn.TreeSpecEngine(t, d, CFG3_TREE, max_batch=1, max_seq=256, max_new_tokens=160)
    toks, st = eng.generate(g["prompt"], 128)
    np.testing.assert_array_equal(toks[:, :g["a_greedy"].shape[1]], g["a_greedy"])
    t_cfg, t_sd, d_cfg, d_sd = variant_b()
    t2, d2 = build(t_cfg, t_sd), build(d_cfg, d_sd)
    rounds = {}
    for name, tree in (("cfg3", CFG3_TREE), ("chain", [-1, 0, 1]), ("wide", [-1, -1, -1, -1, -1, -1])):
        eng = vn.TreeSpecEngine(t2, d2, tree, max_batch=1, max_seq=256, max_new_tokens=128)
        toks, st = eng.generate(g["prompt"], 96)
        np.testing.assert_array_equal(toks[:, :g["b_greedy"].shape[1]], g["b_greedy"])
        rounds[name] = st["rounds"]
    assert rounds["cfg3"] <= rounds["chain"] < 96              # the tree never needs more rounds than its own first path
    # a batch of ragged prompts (left as they are: each row its own length is not supported by prefill, so equal
    # lengths, different contents) against per-request chain decoding
    rng = np.random.default_rng(3)
    prompts = rng.integers(0, 256, (4, 19))
    eng = vn.TreeSpecEngine(t2, d2, CFG3_TREE, max_batch=4, max_seq=256, max_new_tokens=64)
    toks, _ = eng.generate(prompts, 40)
    for b in range(4):
        want = t2.generate(prompts[b:b + 1], max_new_tokens=40, temperature=0.0, draft=d2, k=3)
        np.testing.assert_array_equal(toks[b:b + 1, :want.shape[1]], want)
    with pytest.raises(ValueError):
        vn.TreeSpecEngine(t2, d2, [-1, 2, 0], max_batch=1, max_seq=64)
    with pytest.raises(ValueError):
        vn.TreeSpecEngine(t2, d2, [-1, -1, 0, 1, 0], max_batch=1, max_seq=64)


def test_tree_engine_round_with_more_than_256_rows_in_a_graph():
    """16 requests x 17 tree rows = 272 rows per target forward: beyond the 256-row decode path, so the captured round
    holds the many-row GEMM route (row segments filled by a kernel, nothing copied from the host while capturing).
    The replayed graph commits exactly what the eager rounds commit."""
    import versenext_b200 as vn
    cfg = hd64_cfg()
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=61, gate_std=1.0).items()}
    dcfg = hd64_cfg(n_layer=1, layer_pattern=["trisparse"])
    dsd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(dcfg, seed=62, gate_std=1.0).items()}
    dsd["tok_emb.weight"] = sd["tok_emb.weight"]
    t, d = build(cfg, sd, "bf16"), build(dcfg, dsd, "bf16")
    prompts = np.random.default_rng(9).integers(0, 384, (16, 23))
    outs = []
    for graph in (True, False):
        eng = vn.TreeSpecEngine(t, d, CFG3_TREE, max_batch=16, max_seq=160, max_new_tokens=48, graph=graph)
        toks, st = eng.generate(prompts, 24)
        outs.append(toks[:, :23 + 24])
        assert st["rounds"] >= 6
    np.testing.assert_array_equal(outs[0], outs[1])
    t.check()
    d.check()


def test_continuous_batching_serves_ragged_requests():
    """Seven requests of different prompt lengths and token budgets on three slots: a request leaves its slot when it
    is done and the next one is prefilled into it; every request's tokens equal its own greedy generation."""
    import versenext_b200 as vn
    t_cfg, t_sd, d_cfg, d_sd = variant_b()
    t, d = build(t_cfg, t_sd), build(d_cfg, d_sd)
    rng = np.random.default_rng(77)
    lens = [5, 17, 9, 30, 2, 12, 21]
    budgets = [20, 7, 33, 12, 25, 1, 16]
    prompts = [rng.integers(0, 256, n).astype(np.int64) for n in lens]
    eng = vn.SpecEngine(t, d, max_batch=3, max_seq=128, k=4, temperature=0.0, bonus=True, max_new_tokens=40)
    got = eng.serve(prompts, budgets, poll_every=2)
    for p, n, out in zip(prompts, budgets, got):
        want = t.generate(p[None], max_new_tokens=n, temperature=0.0)[0, len(p):]
        np.testing.assert_array_equal(out, want)
    # EOS: a request stops at its first EOS token, which is kept
    eos = int(got[2][10])
    got2 = eng.serve(prompts, budgets, eos_id=eos, poll_every=3)
    for p, n, full, out in zip(prompts, budgets, got, got2):
        hit = np.flatnonzero(full == eos)
        want = full[:hit[0] + 1] if hit.size else full
        np.testing.assert_array_equal(out, want)
    with pytest.raises(ValueError):
        eng.serve([np.array([1])], 4)
    with pytest.raises(IndexError):
        eng.admit(5, prompts[0])


def test_a_bounded_wait_that_runs_out_is_reported_not_fatal():
    """Failure detection on the device without a fault: a wait on a barrier that nothing ever completes gives up
    after the (shortened) limit, the model's status turns into RuntimeError, and the context keeps working."""
    import ctypes as C
    cfg = hd64_cfg()
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=29, gate_std=1.0).items()}
    m = build(cfg, sd, "bf16")
    lib, ctx = m.ctx.lib, m.ctx
    toks = np.random.default_rng(1).integers(0, 384, (2, 12))
    cache = m.new_cache(2, 64)
    before = m.forward_cached(toks, cache).numpy()
    m.check()                                                   # clean so far
    ctx._check(lib.vn_model_set_wait_limit(m.handle, 2_000_000))          # about a millisecond
    try:
        waited = C.c_int64()
        ctx._check(lib.vn_model_probe_wait(m.handle, C.byref(waited)))
        assert 2_000_000 <= waited.value < 200_000_000
        with pytest.raises(RuntimeError):
            m.check()
    finally:
        ctx._check(lib.vn_model_set_wait_limit(m.handle, 0))
    m.check()                                                   # the condition was cleared by reporting it
    cache.reset()
    np.testing.assert_array_equal(m.forward_cached(toks, cache).numpy(), before)   # same GPU, same answers
