"""Generate the golden fixtures in this folder from the REAL reference.

Run once, in a container that has the reference checkout:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference [fixture names ...]

It imports the reference's own classes (verse_torch, verse_nex), feeds them
seeded inputs and stores inputs + outputs as small .npz files.  The tests
never import the reference; they read these files.
"""

from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("VERSENEXT_REFERENCE", "reference")
sys.path[:0] = [os.path.join(REF, "packages", "verse_torch"),
                os.path.join(REF, "packages", "verse_nex"), REPO]

from verse_torch import Tensor, no_grad  # noqa: E402
from verse_torch.device import NumpyBackend  # noqa: E402
from verse_torch import quantize as rq  # noqa: E402
from verse_nex import SpeculativeDecoder, VerseNexLM  # noqa: E402

from oracle import model as OM  # noqa: E402


def save(name, **arrs):
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrs)
    print(f"wrote {name}: {os.path.getsize(path) / 1024:.1f} KiB")


# ---------------------------------------------------------------------------
# 1. SpeculativeDecoder with a logits-table target
# ---------------------------------------------------------------------------

class TableModel:
    """Target whose logits at position t are row t of a fixed table."""

    def __init__(self, table, as_tuple):
        self.table = table
        self.as_tuple = as_tuple

    def __call__(self, idx):
        ids = np.asarray(idx.data)
        B, T = ids.shape
        lg = np.broadcast_to(self.table[None, :T], (B, T, self.table.shape[1])).astype(np.float32).copy()
        t = Tensor(lg, requires_grad=False)
        hid = Tensor(np.zeros((B, T, 8), dtype=np.float32), requires_grad=False)
        return (t, hid) if self.as_tuple else t


def gen_spec():
    rng = np.random.default_rng(11)
    out = {}
    V, D = 24, 8
    cases = []
    for ci, (k, T_ctx, n_match) in enumerate([(4, 3, 4), (4, 3, 2), (4, 5, 0), (2, 1, 1), (8, 6, 5), (1, 4, 1), (6, 2, 6)]):
        dec = SpeculativeDecoder(dim=D, vocab_size=V, num_draft_heads=k)
        heads = [rng.normal(0, 1, (V, D)).astype(np.float32) for _ in range(k)]
        for h, w in zip(dec.draft_heads, heads):
            h.weight.data = w.copy()
        hidden = rng.normal(0, 1, (2, 3, D)).astype(np.float32)
        draft, dlogits = dec.draft(Tensor(hidden, requires_grad=False))
        table = rng.normal(0, 1, (T_ctx + k + 2, V)).astype(np.float32)
        # make the target agree with row 0's draft on the first n_match positions
        for i in range(k):
            tok = int(draft[0, i]) if i < n_match else (int(draft[0, i]) + 1 + ci) % V
            table[T_ctx - 1 + i, tok] = 50.0
        ctx = rng.integers(0, V, (2, T_ctx)).astype(np.int64)
        model = TableModel(table, as_tuple=bool(ci % 2))
        mask, pred = dec.verify(draft, model, ctx)
        toks, ok, new_ctx = dec.verify_then_commit(draft, model, ctx, max_redraft_rounds=ci % 2)
        p = f"c{ci}_"
        out.update({p + "heads": np.stack(heads), p + "hidden": hidden, p + "draft": draft,
                    p + "draft_logits": np.stack([l.data for l in dlogits]),
                    p + "table": table, p + "ctx": ctx, p + "mask": mask, p + "pred": pred,
                    p + "tokens": np.asarray(toks, dtype=np.int64), p + "all_ok": np.asarray(ok),
                    p + "new_ctx": new_ctx})
        cases.append(ci)
    out["cases"] = np.asarray(cases)
    save("spec_reference.npz", **out)


# ---------------------------------------------------------------------------
# 2/3. Model forward + greedy / speculative streams
# ---------------------------------------------------------------------------

def ref_model(cfg: OM.Config, sd=None, seed=None):
    kw = cfg.to_dict()
    kw.pop("embedding_scale")
    if seed is not None:
        np.random.seed(seed)
    m = VerseNexLM(**kw)
    if sd is not None:
        ref_sd = m.state_dict()
        assert set(ref_sd) == set(OM.param_shapes(cfg)), "state_dict names differ from the reference"
        for n, v in ref_sd.items():
            assert tuple(v.shape) == tuple(sd[n].shape), n
        m.load_state_dict({n: np.array(v) for n, v in sd.items()})
        if cfg.tie_weights:
            assert m.head.weight is m.tok_emb.weight
    m.eval()
    return m


def ref_forward(m, cfg, tokens):
    with no_grad():
        if not cfg.embedding_scale:
            return np.asarray(m(Tensor(tokens.astype(np.int64))).data)
        x = m.tok_emb(Tensor(tokens.astype(np.int64))) * float(np.sqrt(cfg.dim))
        for blk in m.blocks:
            x, _ = blk(x, position_offset=0, kv_cache=None)
        return np.asarray(m.head(m.norm(x)).data)


def ref_greedy(m, cfg, prompt, n_new):
    cur = prompt.copy()
    for _ in range(n_new):
        lg = ref_forward(m, cfg, cur)[:, -1]
        cur = np.concatenate([cur, np.argmax(lg, -1)[:, None]], axis=1)
    return cur


def ref_speculative(target, t_cfg, draft, d_cfg, prompt, k, n_new):
    """Draft model proposes k greedy tokens; the reference SpeculativeDecoder verifies and commits."""
    dec = SpeculativeDecoder(dim=t_cfg.dim, vocab_size=t_cfg.vocab_size, num_draft_heads=k)
    ctx = prompt.copy()
    rounds = accepted = 0
    goal = prompt.shape[1] + n_new

    def target_fn(idx):
        return Tensor(ref_forward(target, t_cfg, np.asarray(idx.data)), requires_grad=False)

    while ctx.shape[1] < goal:
        d = ctx.copy()
        for _ in range(k):
            lg = ref_forward(draft, d_cfg, d)[:, -1]
            d = np.concatenate([d, np.argmax(lg, -1)[:, None]], axis=1)
        toks, ok, ctx = dec.verify_then_commit(d[:, ctx.shape[1]:], target_fn, ctx, max_redraft_rounds=0)
        rounds += 1
        accepted += len(toks) - (0 if ok else 1)
    return ctx[:, :goal], rounds, accepted


def gen_small():
    out = {}
    prompt = np.random.default_rng(0).integers(0, 256, (1, 32)).astype(np.int64)
    # (a) reference-initialised cfg1 (np.random.seed(0) before each constructor)
    t_cfg = OM.small_config()
    d_cfg = OM.small_config(n_layer=1)
    target = ref_model(t_cfg, seed=0)
    draft = ref_model(d_cfg, seed=0)
    t_sd = {n: np.array(v) for n, v in target.state_dict().items()}
    d_sd = {n: np.array(v) for n, v in draft.state_dict().items()}
    for n, v in t_sd.items():
        out["a_t." + n] = v
    for n, v in d_sd.items():
        out["a_d." + n] = v
    out["prompt"] = prompt
    out["a_logits"] = ref_forward(target, t_cfg, prompt)
    out["a_greedy"] = ref_greedy(target, t_cfg, prompt, 128)
    s, r, a = ref_speculative(target, t_cfg, draft, d_cfg, prompt, 4, 128)
    out["a_spec"], out["a_rounds"], out["a_accepted"] = s, np.asarray(r), np.asarray(a)
    print("cfg1 (reference init): rounds", r, "accepted", a, "stream==greedy", np.array_equal(s, out["a_greedy"]),
          "distinct", len(np.unique(s[0, 32:])))

    # (b) non-degenerate: seeded oracle init, untied head, larger init, random gates
    t_cfg2 = OM.small_config(tie_weights=False, init_std=0.2)
    d_cfg2 = OM.small_config(n_layer=1, tie_weights=False, init_std=0.2)
    t_sd2 = OM.init_state_dict(t_cfg2, seed=101, gate_std=1.0)
    d_sd2 = OM.init_state_dict(d_cfg2, seed=102, gate_std=1.0)
    # draft shares the target's embedding and head so that it agrees sometimes
    # and its single block is the target's block 0 plus noise
    d_sd2["tok_emb.weight"] = t_sd2["tok_emb.weight"]
    d_sd2["head.weight"] = t_sd2["head.weight"]
    for n in list(d_sd2):
        if n.startswith("blocks.0.") and not n.endswith("norm1.weight") and not n.endswith("norm2.weight"):
            d_sd2[n] = (t_sd2[n] + 0.15 * d_sd2[n]).astype(np.float32)
    target2 = ref_model(t_cfg2, t_sd2)
    draft2 = ref_model(d_cfg2, d_sd2)
    out["b_logits"] = ref_forward(target2, t_cfg2, prompt)
    out["b_greedy"] = ref_greedy(target2, t_cfg2, prompt, 96)
    s, r, a = ref_speculative(target2, t_cfg2, draft2, d_cfg2, prompt, 4, 96)
    out["b_spec"], out["b_rounds"], out["b_accepted"] = s, np.asarray(r), np.asarray(a)
    print("cfg1 variant (seeded, untied): rounds", r, "accepted", a, "stream==greedy",
          np.array_equal(s, out["b_greedy"]), "distinct", len(np.unique(s[0, 32:])))
    save("model_small.npz", **out)


def gen_mini():
    """Mate-shaped miniature: rope, no alibi, GQA, MoD every 4th layer, tied, embedding scale."""
    out = {}
    cfg = OM.mate_config(vocab_size=512, dim=64, n_layer=4, n_head=4, n_kv_head=2, window_size=16,
                         num_global_tokens=8, max_seq_len=128, init_std=0.1)
    sd = OM.init_state_dict(cfg, seed=7, gate_std=1.0)
    m = ref_model(cfg, sd)
    toks = np.random.default_rng(5).integers(0, 512, (2, 40)).astype(np.int64)
    out["tokens"] = toks
    out["logits"] = ref_forward(m, cfg, toks)
    # window-limited + no-scale variant, batch 1, longer than 2 windows
    cfg2 = OM.mate_config(vocab_size=512, dim=64, n_layer=4, n_head=4, n_kv_head=2, window_size=16,
                          num_global_tokens=8, max_seq_len=128, init_std=0.1, embedding_scale=False,
                          use_alibi=True)
    m2 = ref_model(cfg2, sd)
    out["logits_alibi_rope"] = ref_forward(m2, cfg2, toks[:1])
    # the reference's own incremental path: blocks with kv_cache (prefill 30, then 10 more)
    with no_grad():
        x = m.tok_emb(Tensor(toks[:, :30])) * float(np.sqrt(cfg.dim))
        caches = []
        for blk in m.blocks:
            x, st = blk(x, position_offset=0, kv_cache=None)
            caches.append(st["kv_cache"])
        x = m.tok_emb(Tensor(toks[:, 30:])) * float(np.sqrt(cfg.dim))
        for blk, c in zip(m.blocks, caches):
            x, st = blk(x, position_offset=0, kv_cache=c)
        out["logits_incremental"] = np.asarray(m.head(m.norm(x)).data)
    save("model_mini.npz", **out)


# ---------------------------------------------------------------------------
# 4. quantisation, 5. backend ops
# ---------------------------------------------------------------------------

def gen_quant():
    rng = np.random.default_rng(21)
    w = rng.normal(0, 0.05, (48, 64)).astype(np.float32)
    w[3] = 0.0
    x = rng.normal(0, 1, (5, 64)).astype(np.float32)
    q8, s8 = rq.quantize_int8(w)
    p4, s4 = rq.quantize_int4(w)
    out = dict(w=w, x=x, q8=q8, s8=s8, p4=p4, s4=s4,
               y4=rq.matmul_int4(x, p4, s4, w.shape))
    from verse_torch.vnnn import Linear
    lin = Linear(64, 48, bias=True)
    lin.weight.data = w.copy()
    lin.bias.data = rng.normal(0, 0.1, (48,)).astype(np.float32)
    out["bias"] = np.array(lin.bias.data)
    for qt in ("int8", "int4"):
        for cache in (True, False):
            ql = rq.QuantizedLinear(lin, qtype=qt, cache_fp32=cache)
            out[f"ql_{qt}_{int(cache)}"] = np.asarray(ql.forward(Tensor(x)).data)
        out[f"ql_{qt}_fused"] = np.asarray(ql.forward_fused(Tensor(x)).data)
    save("quant_reference.npz", **out)


def gen_backend():
    rng = np.random.default_rng(31)
    be = NumpyBackend()
    a = rng.normal(0, 1, (3, 7, 16)).astype(np.float32)
    b = rng.normal(0, 1, (3, 16, 5)).astype(np.float32)
    w = rng.normal(0, 1, (12, 16)).astype(np.float32)
    bias = rng.normal(0, 1, (12,)).astype(np.float32)
    g = rng.normal(1, 0.1, (16,)).astype(np.float32)
    beta = rng.normal(0, 0.1, (16,)).astype(np.float32)
    q = rng.normal(0, 1, (2, 4, 6, 8)).astype(np.float32)
    k = rng.normal(0, 1, (2, 4, 9, 8)).astype(np.float32)
    v = rng.normal(0, 1, (2, 4, 9, 8)).astype(np.float32)
    mask = np.where(rng.random((6, 9)) < 0.3, -1e9, 0.0).astype(np.float32)
    mask[:, 0] = 0.0
    cos, sin = OM.rope_table(8, 6)
    save("backend_reference.npz", a=a, b=b, w=w, bias=bias, g=g, beta=beta, q=q, k=k, v=v, mask=mask,
         cos=cos, sin=sin,
         matmul=be.matmul(a, b), linear=be.linear(a, w, bias), linear_nobias=be.linear(a, w),
         softmax=be.softmax(a, dim=-1), softmax_d1=be.softmax(a, dim=1),
         layernorm=be.layernorm(a, g, beta, eps=1e-5), rmsnorm=be.rmsnorm(a, g, eps=1e-6),
         rope_full=be.rope(q, cos, sin), rope_half=be.rope(q, cos[:, :4], sin[:, :4]),
         attention=be.attention(q, k, v), attention_mask=be.attention(q, k, v, mask))


# ---------------------------------------------------------------------------
# 6. Sampling: the probability vectors the reference's two samplers draw from
# ---------------------------------------------------------------------------

class _RecordingRng:
    """Stands in for the NumPy generator inside the reference's samplers: keeps the probability vector
    that `choice` is asked to draw from and returns index 0."""

    def __init__(self):
        self.calls = []

    def choice(self, n, p=None, **kw):
        self.calls.append((int(n) if np.isscalar(n) else len(n), np.array(p, copy=True)))
        return 0


def gen_sampling():
    """`Sampler.sample` (verse_infra/verse_inference/sampler.py:86-138: threshold rule, ties kept) and
    `VerseNexLM._generate_with_logits` (verse_nex/cometspark.py:892-911: argpartition rule, exactly k kept):
    both run unmodified; the generator they draw with is replaced by a recorder."""
    sys.path.insert(0, os.path.join(REF, "packages", "verse_infra"))
    from verse_infra.verse_inference.sampler import Sampler
    import verse_nex.cometspark as cs
    rng = np.random.default_rng(41)
    V = 1000
    rows = rng.normal(0, 2.0, (6, V)).astype(np.float32)
    rows[2, rng.choice(V, 7, replace=False)] = rows[2].max() + 1.0       # seven-way tie on top
    rows[3, rng.choice(V, 30, replace=False)] = np.sort(rows[3])[-10]    # ties exactly at the 10th largest
    rows[4] = np.round(rows[4])                                          # few distinct values
    cases = [(1.0, 0), (0.8, 50), (0.8, 10), (1.3, 5), (0.5, 1), (1.0, 2000)]
    out = {"rows": rows, "temperature": np.array([c[0] for c in cases], np.float32),
           "top_k": np.array([c[1] for c in cases], np.int64)}
    for ci, (T, k) in enumerate(cases):
        for ri in range(rows.shape[0]):
            smp = Sampler(temperature=T, top_k=k, top_p=1.0, seed=0)
            rec = _RecordingRng()
            smp._rng = rec
            smp.sample(rows[ri])
            out[f"sampler_c{ci}_r{ri}"] = rec.calls[0][1].astype(np.float64)
    # the generate path: a real (tiny) model whose forward is replaced by the fixed logits rows
    cfg = OM.small_config(vocab_size=V)
    m = ref_model(cfg, seed=3)
    for ci, (T, k) in enumerate(cases):
        rec = _RecordingRng()
        real_rng = np.random.default_rng
        np.random.default_rng = lambda *a, **kw: rec
        m.forward = lambda idx: Tensor(np.broadcast_to(rows[:, None, :], (rows.shape[0], idx.data.shape[1], V)).copy(),
                                       requires_grad=False)
        try:
            m._generate_with_logits(np.zeros((rows.shape[0], 3), np.int64), 1, T, (k if k > 0 else None))
        finally:
            np.random.default_rng = real_rng
        # with top-k the code draws an index into top_idx[b]; re-derive top_idx exactly as the code does
        scaled = rows / max(T, 1e-8)
        for ri in range(rows.shape[0]):
            full = np.zeros(V, np.float64)
            if k > 0:
                kk = min(k, V)
                top_idx = np.argpartition(-scaled, kth=kk - 1, axis=-1)[:, :kk]
                full[top_idx[ri]] = rec.calls[ri][1]
            else:
                full[:] = rec.calls[0][1][ri] if rec.calls[0][1].ndim == 2 else rec.calls[ri][1]
            out[f"generate_c{ci}_r{ri}"] = full
    save("sampling_reference.npz", **out)


# ---------------------------------------------------------------------------
# 7. The recurrent decoding path and the greedy `generate` built on it, longer than the window
# ---------------------------------------------------------------------------

def gen_recurrent():
    """`forward_recurrent` token by token (cometspark.py:737-767; attention state trimmed to the last
    `window_size` keys, tri_sparse_attn.py:676-684) and `generate` with its defaults (greedy, :817-818, which
    feeds the last prompt token a second time, :848-856) for sequences longer than the window, with the ALiBi
    path on (small config) and with RoPE (miniature mate config)."""
    out = {}
    for tag, cfg, seed in (("alibi", OM.small_config(tie_weights=False, init_std=0.2), 201),
                           ("rope", OM.mate_config(vocab_size=512, dim=64, n_layer=2, n_head=4, n_kv_head=2,
                                                   window_size=16, num_global_tokens=8, max_seq_len=256,
                                                   init_std=0.2, num_dense_parts=2, num_experts_per_part=2, top_k=1,
                                                   layer_pattern=["trisparse", "trisparse"], embedding_scale=False),
                            202)):
        sd = OM.init_state_dict(cfg, seed=seed, gate_std=1.0)
        m = ref_model(cfg, sd)
        for n, v in sd.items():
            out[f"{tag}.{n}"] = v
        W = cfg.window_size
        T = 2 * W + 9
        toks = np.random.default_rng(seed).integers(0, cfg.vocab_size, (2, T)).astype(np.int64)
        states, rows = None, []
        with no_grad():
            for t in range(T):
                lg, states = m.forward_recurrent(Tensor(toks[:, t:t + 1]), states)
                rows.append(np.asarray(lg.data)[:, 0])
        out[f"{tag}_tokens"] = toks
        out[f"{tag}_recurrent_logits"] = np.stack(rows, axis=1).astype(np.float32)      # (B, T, V)
        out[f"{tag}_generate"] = m.generate(toks[:, :W + 5], max_new_tokens=W + 7)
        out[f"{tag}_generate_eos"] = m.generate(toks[:1, :6], max_new_tokens=12, eos_id=int(out[f"{tag}_generate"][0, W + 6]))
        print(tag, "recurrent", out[f"{tag}_recurrent_logits"].shape, "generate", out[f"{tag}_generate"].shape,
              "distinct", len(np.unique(out[f"{tag}_generate"][0, W + 5:])))
    save("recurrent_reference.npz", **out)


# ---------------------------------------------------------------------------
# 8. A model written by the reference into its .vn container (both weight formats)
# ---------------------------------------------------------------------------

def gen_vn():
    import verse_torch.vn_format as vf
    cfg = OM.mate_config(vocab_size=96, dim=32, n_layer=2, n_head=2, n_kv_head=1, window_size=8, num_global_tokens=4,
                         max_seq_len=64, init_std=0.2, num_dense_parts=2, num_experts_per_part=2, top_k=1,
                         expert_hidden=64, embedding_scale=False)
    sd = OM.init_state_dict(cfg, seed=301, gate_std=1.0)
    m = ref_model(cfg, sd)
    toks = np.random.default_rng(301).integers(0, 96, (2, 19)).astype(np.int64)
    out = {"tokens": toks, "logits": ref_forward(m, cfg, toks)}
    for n, v in m.state_dict().items():
        out["sd." + n] = np.array(v)
    m.save_vn(os.path.join(HERE, "model_tiny_st.vn"))
    had = vf._HAS_SAFETENSORS
    vf._HAS_SAFETENSORS = False                  # the writer's fallback: one .npy member per tensor
    try:
        m.save_vn(os.path.join(HERE, "model_tiny_npz.vn"))
    finally:
        vf._HAS_SAFETENSORS = had
    for f in ("model_tiny_st.vn", "model_tiny_npz.vn"):
        print(f"wrote {f}: {os.path.getsize(os.path.join(HERE, f)) / 1024:.1f} KiB")
    save("vn_reference.npz", **out)
    # a model of delta attention layers through the same writer (names like blocks.0.attn.gmla.w_kv_down.weight,
    # anchor_interval / latent_dim in config.yml)
    from oracle import delta as OD
    # (the writer takes window_size / use_alibi / ... from block 0's attention, cometspark.py:1238-1243, which only a
    # TriSparse block has, and does not store anchor_interval / latent_dim: block 0 is TriSparse, those two keep
    # their defaults)
    cfg = OM.Config(vocab_size=64, dim=32, n_layer=3, n_head=2, n_kv_head=1, layer_pattern=["trisparse", "vda", "dsa"],
                    window_size=8, num_global_tokens=3, use_alibi=False, use_rope=True, max_seq_len=64, init_std=0.2)
    sd = OM.init_state_dict(cfg, seed=302, gate_std=1.0)
    m = ref_model(cfg, sd)
    toks = np.random.default_rng(302).integers(0, 64, (2, 21)).astype(np.int64)
    out = {"tokens": toks, "logits": ref_forward(m, cfg, toks)}       # the weights are init_state_dict(cfg, seed=302)
    m.save_vn(os.path.join(HERE, "model_tiny_delta.vn"))
    print(f"wrote model_tiny_delta.vn: {os.path.getsize(os.path.join(HERE, 'model_tiny_delta.vn')) / 1024:.1f} KiB")
    save("vn_delta_reference.npz", **out)


# ---------------------------------------------------------------------------
# 9. Delta attention family (vda / dsa / kda / gmla layers)
# ---------------------------------------------------------------------------

def gen_delta():
    """Whole-sequence logits of models built from the delta attention kinds: a short case per layout (every class
    on its full-matrix route) and one of 1100 tokens (every class beyond its 1024-key switch)."""
    from verse_nex.delta_attention import build_verse_delta_pattern
    out = {}
    for n in (1, 5, 6, 9, 10, 14):
        out[f"pattern_{n}"] = np.array(build_verse_delta_pattern(n))
    from oracle import delta as OD
    # A: rope, GQA, one layer of every kind
    cfg, sd = OD.golden_case("a")
    m = ref_model(cfg, sd)
    toks = np.random.default_rng(32).integers(0, 96, (2, 40)).astype(np.int64)
    out["a_tokens"] = toks
    out["a_logits"] = ref_forward(m, cfg, toks)
    out["a_greedy"] = ref_greedy(m, cfg, toks[:, :8], 24)
    # B: no rope, multi-head, a latent narrower than K | V, anchors wider apart than the window
    cfg, sd = OD.golden_case("b")
    m = ref_model(cfg, sd)
    toks = np.random.default_rng(34).integers(0, 80, (3, 33)).astype(np.int64)
    out["b_tokens"] = toks
    out["b_logits"] = ref_forward(m, cfg, toks)
    # C: 1100 tokens -- dense routes fall back to window (+ sinks), KDA goes chunk-wise with its anchors concatenated
    cfg, sd = OD.golden_case("c")
    m = ref_model(cfg, sd)
    toks = np.random.default_rng(36).integers(0, 64, (1, 1100)).astype(np.int64)
    rows = np.array([0, 1, 39, 40, 47, 48, 95, 96, 500, 960, 1023, 1024] + list(range(1088, 1100)))
    lg = ref_forward(m, cfg, toks)
    out["c_tokens"] = toks
    out["c_rows"] = rows
    out["c_logits"] = lg[:, rows]
    # the same model at 1024 tokens is still on the full-matrix routes
    lg = ref_forward(m, cfg, toks[:, :1024])
    out["c_logits_1024"] = lg[:, rows[:11]]
    # the one-token route of the same model (cometspark.py:737-767 -> forward_recurrent of every class): fed token by
    # token past 1024 keys.  There DSA keeps its dense soft-max and KDA its plain window | anchor mask (:580-616,
    # :780-803); only GMLA switches to the window (:1059-1069)
    T = 1040
    r_rows = np.array([0, 1, 47, 48, 500, 1023, 1024, 1025, 1039])
    states, keep = None, []
    with no_grad():
        for t in range(T):
            lg, states = m.forward_recurrent(Tensor(toks[:, t:t + 1]), states)
            if t in r_rows:
                keep.append(np.asarray(lg.data)[:, 0])
    out["c_recurrent_rows"] = r_rows
    out["c_recurrent_logits"] = np.stack(keep, axis=1).astype(np.float32)
    # generate with its defaults (greedy on the one-token route, the last prompt token fed twice) on model a
    cfg, sd = OD.golden_case("a")
    m = ref_model(cfg, sd)
    out["a_generate_default"] = m.generate(out["a_tokens"][:, :8], max_new_tokens=24)
    save("delta_reference.npz", **out)


if __name__ == "__main__":
    only = set(sys.argv[2:])          # e.g. `make_golden.py /path/to/reference sampling recurrent`
    for name, fn in (("spec", gen_spec), ("small", gen_small), ("mini", gen_mini), ("quant", gen_quant),
                     ("backend", gen_backend), ("sampling", gen_sampling), ("recurrent", gen_recurrent), ("vn", gen_vn), ("delta", gen_delta)):
        if not only or name in only:
            fn()
