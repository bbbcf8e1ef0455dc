"""Generate the golden fixtures in this folder from the REAL reference.

Run once, in a container that has the reference checkout:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

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


if __name__ == "__main__":
    gen_spec()
    gen_small()
    gen_mini()
    gen_quant()
    gen_backend()
