"""NumPy restatement of the VerseNext Delta Attention family (test infrastructure, CPU).

Follows verse_nex/delta_attention.py of the reference:
  * shared projections, RoPE, GQA repeat      _DeltaAttentionBase.forward        :238-281
  * DSA   head-gated dense | window + sinks   DSAAttention._attend               :555-574
          dense causal                         :470-486, window :492-538, sinks :451-459, :540-549
  * KDA   window | anchors in one soft-max    KDAAttention._anchor_window_forward :678-698
          long sequences, chunk-wise           :704-768 (the anchors are concatenated behind the window slice)
  * GMLA  latent K / V + head gate            GMLAAttention.forward              :876-930, window :948-992
  * VDA   sigmoid-gated sum of the three      VDAAttention.forward               :1144-1176
  * layer pattern                              build_verse_delta_pattern          :1218-1247

What is restated is the WHOLE-SEQUENCE forward (no kv_cache, position_offset 0), which is what
`SpeculativeDecoder.verify` runs (speculative.py:202-213).  Like `oracle.model.attention`, the functions here also
accept a cache and a tree parent array; both are defined so that the result equals the whole-sequence forward over
the same tokens: masks are built from absolute positions.  (The reference's own kv_cache route is not that function:
its dense masks compare local query indices with global key indices, :477-479, and GMLA rebuilds K / V from the new
latents only, :894-896.)

Length switch: every class leaves its full-matrix route when the key count exceeds `_MAX_T` = 1024 (:406, :640,
:825).  With a cache the key count of a chain is cached + new positions, of a tree node its own position + 1 -- the
same convention `oracle.model.attention` uses for the ALiBi switch.

KDA beyond 1024 keys: the chunk-wise route scores the window slice [k_lo, k_hi) of the query's chunk AND all anchors,
concatenated (:742-743), so an anchor that also lies in the slice enters the soft-max twice.  `kda_multiplicity`
returns that count per (query, key); the soft-max below weights exp(score) by it.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32
MAX_T = 1024          # delta_attention.py:406, :640, :825
DELTA_KINDS = ("vda", "dsa", "kda", "gmla")


def build_verse_delta_pattern(n_layer: int) -> list:
    """delta_attention.py:1218-1247."""
    if n_layer < 1:
        raise ValueError(f"n_layer must be >= 1, got {n_layer}")
    if n_layer < 6:
        return ["vda"] * n_layer
    if n_layer < 10:
        return ["vda"] * 4 + ["gmla"] * (n_layer - 4)
    return ["vda"] * 4 + ["gmla"] * (n_layer - 6) + ["dsa"] * 2


def sub_param_shapes(cfg, kind, include_proj=True) -> dict:
    """Parameter names (relative to the attention module) -> shapes of one DSA / KDA / GMLA module."""
    D, hd = cfg.dim, cfg.head_dim
    qd, kvd = cfg.n_head * hd, cfg.n_kv_head * hd
    s = {"wq.weight": (qd, D)}
    if kind == "gmla":
        lat = cfg.latent_dim if cfg.latent_dim is not None else kvd
        s["w_kv_down.weight"] = (lat, D)
        s["w_k_up.weight"] = (kvd, lat)
        s["w_v_up.weight"] = (kvd, lat)
        s["head_gate_logits"] = (cfg.n_head,)
    else:
        s["wk.weight"] = (kvd, D)
        s["wv.weight"] = (kvd, D)
        if kind == "dsa":
            s["head_gate_logits"] = (cfg.n_head,)
            s["global_tokens.weight"] = (cfg.num_global_tokens, D)
    if include_proj:
        s["proj.weight"] = (D, qd)
    return s


def attn_param_shapes(cfg, kind) -> dict:
    """Names relative to `blocks.i.attn.` for a layer of a delta kind."""
    if kind != "vda":
        return sub_param_shapes(cfg, kind)
    s = {"gate_logits": (3,), "proj.weight": (cfg.dim, cfg.dim)}
    for sub in ("dsa", "kda", "gmla"):
        for n, shp in sub_param_shapes(cfg, sub, include_proj=False).items():
            s[f"{sub}.{n}"] = shp
    return s


def _sigmoid(x):
    return (0.5 * (1.0 + np.tanh(0.5 * np.asarray(x, F32)))).astype(F32)   # _np_sigmoid :68-70 (== Tensor.sigmoid)


def _softmax_masked(scores, mask):
    """softmax(scores + where(mask, 0, -1e9)) as the reference builds it (:480-483)."""
    s = scores + np.where(mask, 0.0, -1e9).astype(F32)
    m = np.max(s, axis=-1, keepdims=True)
    e = np.exp(s - m)
    return (e / np.sum(e, axis=-1, keepdims=True)).astype(F32)


def kda_multiplicity(pos, key_pos, visible, window, interval):
    """How often key j enters query t's soft-max on the chunk-wise KDA route (:704-768): once through the window
    slice of t's chunk when it is in the window or an anchor inside the slice, once more through the anchor list."""
    pos = np.asarray(pos)[:, None]
    kp = np.asarray(key_pos)[None, :]
    causal = visible & (kp <= pos)
    k_lo = np.maximum(0, (pos // window) * window - window + 1)
    anchor = (kp % interval) == 0
    in_win = (pos - kp) < window
    in_slice = causal & (kp >= k_lo) & (in_win | anchor)
    return in_slice.astype(np.int64) + (causal & anchor).astype(np.int64)


def _geometry(cache_len, T, parents, recurrent=False):
    from .model import tree_depths_and_ancestors
    if parents is None:
        depth = np.arange(T)
        vis_new = np.tril(np.ones((T, T), dtype=bool))
    else:
        depth, vis_new = tree_depths_and_ancestors(parents)
    pos = cache_len + depth
    key_pos = np.concatenate([np.arange(cache_len), pos])
    visible = np.zeros((T, cache_len + T), dtype=bool)
    visible[:, :cache_len] = True
    visible[:, cache_len:] = vis_new
    # key count that decides the length switch: the whole call for a chain, a row's own position + 1 for a tree node
    # and on the one-token route (where every token is a call of its own)
    tk_eff = np.full(T, cache_len + T) if (parents is None and not recurrent) else (pos + 1)
    return pos, key_pos, visible, tk_eff


def sub_attention(sd, cfg, prefix, kind, x, cache, parents, rope, recurrent=False):
    """One DSA / KDA / GMLA module without its output projection: head-space output [B, T, H*hd] and the new
    cache {'k', 'v'} (for GMLA the K / V rebuilt from the latents: the same information as the latent cache).

    recurrent=True restates the classes' `forward_recurrent` (one token per call, :294-375, :998-1085), evaluated
    for all T positions at once: every row is its own call, so GMLA's switch to the window looks at the row's own key
    count (:1059), while DSA keeps its dense soft-max (:594-597) and KDA its plain window | anchor mask (:788-799) at
    any length."""
    from .model import linear, apply_rope
    B, T, D = x.shape
    H, hd, n_kv = cfg.n_head, cfg.head_dim, cfg.n_kv_head
    n_rep = H // n_kv
    Tc = 0 if cache is None else cache["k"].shape[1]
    pos, key_pos, visible, tk_eff = _geometry(Tc, T, parents, recurrent)
    q = linear(x, sd[prefix + "wq.weight"]).reshape(B, T, H, hd)
    if kind == "gmla":
        c = linear(x, sd[prefix + "w_kv_down.weight"])
        k = linear(c, sd[prefix + "w_k_up.weight"]).reshape(B, T, n_kv, hd)
        v = linear(c, sd[prefix + "w_v_up.weight"]).reshape(B, T, n_kv, hd)
    else:
        k = linear(x, sd[prefix + "wk.weight"]).reshape(B, T, n_kv, hd)
        v = linear(x, sd[prefix + "wv.weight"]).reshape(B, T, n_kv, hd)
    if cfg.use_rope:
        cos, sin = rope
        q = apply_rope(q, pos, cos, sin)
        k = apply_rope(k, pos, cos, sin)
    if cache is not None:
        k = np.concatenate([cache["k"], k], axis=1)
        v = np.concatenate([cache["v"], v], axis=1)
    new_cache = {"k": k, "v": v}
    kr = np.repeat(k, n_rep, axis=2).transpose(0, 2, 1, 3)
    vr = np.repeat(v, n_rep, axis=2).transpose(0, 2, 1, 3)
    qh = q.transpose(0, 2, 1, 3)
    scale = F32(1.0 / (hd ** 0.5))
    scores = ((qh @ kr.transpose(0, 1, 3, 2)) * scale).astype(F32)          # B,H,T,Tk
    dist = pos[:, None] - key_pos[None, :]
    dense = visible & (dist >= 0)
    win = dense & (dist < cfg.window_size)
    long_row = (tk_eff > MAX_T)[None, None, :, None]
    if recurrent and kind != "gmla":
        long_row = np.zeros_like(long_row)

    if kind == "kda":
        I = cfg.anchor_interval
        anchor = (key_pos % I == 0)[None, :]
        out_short = _softmax_masked(scores, (dense & (win | anchor))[None, None]) @ vr
        if np.any(long_row):
            mult = kda_multiplicity(pos, key_pos, visible, cfg.window_size, I).astype(F32)[None, None]
            s = np.where(mult > 0, scores, F32(-np.inf))
            e = np.exp(s - np.max(s, axis=-1, keepdims=True)) * mult
            out_long = (e / np.sum(e, axis=-1, keepdims=True)).astype(F32) @ vr
            out = np.where(long_row, out_long, out_short)
        else:
            out = out_short
    elif kind == "gmla":
        out_dense = _softmax_masked(scores, dense[None, None]) @ vr
        out_win = _softmax_masked(scores, win[None, None]) @ vr
        gate = _sigmoid(sd[prefix + "head_gate_logits"]).reshape(1, H, 1, 1)
        out = np.where(long_row, out_win, out_dense) * gate
    elif kind == "dsa":
        g = sd[prefix + "global_tokens.weight"]
        n_g = g.shape[0]
        kg = np.repeat(linear(g, sd[prefix + "wk.weight"]).reshape(n_g, n_kv, hd), n_rep, axis=1).transpose(1, 0, 2)
        vg = np.repeat(linear(g, sd[prefix + "wv.weight"]).reshape(n_g, n_kv, hd), n_rep, axis=1).transpose(1, 0, 2)
        sg = (qh @ kg.transpose(0, 2, 1)[None]) * scale
        eg = np.exp(sg - np.max(sg, axis=-1, keepdims=True))
        glob = (eg / np.sum(eg, axis=-1, keepdims=True)).astype(F32) @ vg[None]
        sparse = _softmax_masked(scores, win[None, None]) @ vr + glob
        dense_out = np.where(long_row, sparse, _softmax_masked(scores, dense[None, None]) @ vr)
        gate = _sigmoid(sd[prefix + "head_gate_logits"]).reshape(1, H, 1, 1)
        out = dense_out * gate + sparse * (F32(1.0) - gate)
    else:
        raise ValueError(kind)
    return out.astype(F32).transpose(0, 2, 1, 3).reshape(B, T, H * hd), new_cache


def attention(sd, cfg, prefix, kind, x, cache, parents, rope, recurrent=False):
    """The attention module of a block of kind vda / dsa / kda / gmla (`prefix` ends with 'attn.'): output
    [B, T, D] after the projection, and the new cache (nested per sub-module for vda)."""
    from .model import linear
    if kind != "vda":
        o, c = sub_attention(sd, cfg, prefix, kind, x, cache, parents, rope, recurrent)
        return linear(o, sd[prefix + "proj.weight"]), c
    gate = _sigmoid(sd[prefix + "gate_logits"])
    total, new_cache = None, {}
    for i, sub in enumerate(("dsa", "kda", "gmla")):
        o, c = sub_attention(sd, cfg, prefix + sub + ".", sub, x, None if cache is None else cache[sub], parents, rope,
                             recurrent)
        new_cache[sub] = c
        total = gate[i] * o if total is None else total + gate[i] * o
    return linear(total.astype(F32), sd[prefix + "proj.weight"]), new_cache


def golden_case(tag):
    """(Config, state_dict) of the models behind tests/golden/delta_reference.npz (cases "a", "b", "c")."""
    from . import model as OM
    if tag == "a":      # rope, GQA, one layer of every kind
        cfg = OM.Config(vocab_size=96, dim=64, n_layer=4, n_head=4, n_kv_head=2,
                        layer_pattern=["vda", "gmla", "dsa", "kda"], window_size=8, num_global_tokens=4,
                        anchor_interval=4, use_alibi=False, use_rope=True, max_seq_len=64, init_std=0.1)
        seed = 31
    elif tag == "b":    # no rope, multi-head, a latent narrower than K | V, anchors wider apart than the window
        cfg = OM.Config(vocab_size=80, dim=48, n_layer=3, n_head=3, n_kv_head=3, layer_pattern=["kda", "vda", "gmla"],
                        window_size=6, num_global_tokens=3, anchor_interval=10, latent_dim=24, use_alibi=False,
                        use_rope=False, max_seq_len=64, tie_weights=False, init_std=0.1)
        seed = 33
    elif tag == "c":    # run at 1100 tokens: every class beyond its 1024-key switch
        cfg = OM.Config(vocab_size=64, dim=32, n_layer=4, n_head=2, n_kv_head=1,
                        layer_pattern=["vda", "kda", "gmla", "dsa"], window_size=48, num_global_tokens=5,
                        anchor_interval=40, use_alibi=False, use_rope=True, max_seq_len=2048, init_std=0.15)
        seed = 35
    else:
        raise ValueError(tag)
    return cfg, OM.init_state_dict(cfg, seed=seed, gate_std=1.0)
