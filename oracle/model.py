"""NumPy restatement of the VerseNexLM forward (test infrastructure, CPU).

Follows, function by function, the reference fp32 CPU path:
  * CometSparkNexLM.forward            verse_nex/cometspark.py:670-698
  * CometSparkV05LM embedding scale    spark/src/base_model.py:199-206
  * VerseNexBlock.forward              verse_nex/cometspark.py:215-250
  * TriSparseAttention.forward         verse_nex/tri_sparse_attn.py:536-613
      RoPE table / apply               :169-206   (NeoX half split, fp32 table)
      sink K/V (never rotated)         :223-242
      path A window + causal, -1e9     :341-346, :437-443
      path B sinks                     :461-483
      path C ALiBi, T_k <= 1024        :489-530, :600
      sigmoid gate mix                 :590-608
  * MoDLayer / Router / experts        verse_nex/mod.py:340-387, :142-213, :748-799
  * SwiGLUMLP, RMSNorm, Linear         verse_torch/vnnn.py:801-807, :501-505, :423-430
  * silu = x*0.5*(1+tanh(x/2))         verse_torch/tensor.py:853-856

The reference evaluates path A chunk-wise over padded score tensors; this
restatement evaluates the same masked softmax densely (masked entries get
-1e9 and underflow to exactly 0 in float32, so the two are the same
function).  Unlike the reference's `verify`, which re-runs the whole context
(speculative.py:202-213), `forward` here also accepts a KV cache and a tree
parent array; with `cache=None, parents=None` it is the reference forward.
Pinned against the real reference classes by tests/golden/model_*.npz.
"""

from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import List, Optional

import numpy as np

from . import delta
from .delta import DELTA_KINDS

F32 = np.float32
ALIBI_MAX_T = 1024  # tri_sparse_attn.py:94


@dataclass
class Config:
    """Keyword arguments of CometSparkNexLM.__init__ (cometspark.py:334-364)."""
    vocab_size: int
    dim: int
    n_layer: int
    n_head: int
    n_kv_head: Optional[int] = None
    layer_pattern: Optional[List[str]] = None
    window_size: int = 512
    num_global_tokens: int = 64
    anchor_interval: int = 128
    latent_dim: Optional[int] = None
    use_alibi: bool = True
    use_rope: bool = False
    max_seq_len: int = 2048
    rope_theta: float = 10000.0
    num_dense_parts: int = 5
    num_experts_per_part: int = 8
    top_k: int = 3
    expert_hidden: Optional[int] = None
    tie_weights: bool = True
    mlp_hidden_multiple: int = 4
    init_std: float = 0.02
    embedding_scale: bool = False  # CometSparkV05LM wrapper only

    def __post_init__(self):
        if self.n_kv_head is None:
            self.n_kv_head = self.n_head
        if self.layer_pattern is None:
            self.layer_pattern = ["trisparse"] * self.n_layer
        if len(self.layer_pattern) != self.n_layer:
            raise ValueError("layer_pattern length must equal n_layer")
        if self.expert_hidden is None:
            self.expert_hidden = max(int(self.dim * 8 / 3 / 64) * 64, 64)  # mod.py:687-688

    @property
    def head_dim(self):
        return self.dim // self.n_head

    @property
    def mlp_hidden(self):
        align = 64
        return int((self.mlp_hidden_multiple * self.dim * 2 / 3 + align - 1) // align) * align  # vnnn.py:794

    def to_dict(self):
        return asdict(self)


def mate_config(**over) -> Config:
    """CometSparkV05 factory defaults (spark/src/base_model.py:760-786)."""
    kw = dict(vocab_size=248320, dim=1024, n_layer=20, n_head=16, n_kv_head=8,
              layer_pattern=["mod" if i % 4 == 0 else "trisparse" for i in range(20)],
              window_size=1024, num_global_tokens=128, use_alibi=False, use_rope=True,
              max_seq_len=4096, num_dense_parts=4, num_experts_per_part=4, top_k=2,
              tie_weights=True, embedding_scale=True)
    kw.update(over)
    if "n_layer" in over and "layer_pattern" not in over:
        kw["layer_pattern"] = ["mod" if i % 4 == 0 else "trisparse" for i in range(kw["n_layer"])]
    return Config(**kw)


def small_config(**over) -> Config:
    """The CPU-runnable small configuration: all-trisparse, alibi, no rope, dim 64, vocab 256."""
    kw = dict(vocab_size=256, dim=64, n_layer=2, n_head=4, n_kv_head=2,
              window_size=32, num_global_tokens=4, use_alibi=True, use_rope=False,
              max_seq_len=256, tie_weights=True)
    kw.update(over)
    return Config(**kw)


def param_shapes(cfg: Config) -> dict:
    """Dotted state_dict names -> shapes, as Module.state_dict() yields them (vnnn.py:235-252)."""
    D, hd = cfg.dim, cfg.head_dim
    kv = cfg.n_kv_head * hd
    s = {"tok_emb.weight": (cfg.vocab_size, D), "norm.weight": (D,),
         "head.weight": (cfg.vocab_size, D)}
    for i, kind in enumerate(cfg.layer_pattern):
        p = f"blocks.{i}."
        s[p + "norm1.weight"] = (D,)
        s[p + "norm2.weight"] = (D,)
        if kind in DELTA_KINDS:
            for n, shp in delta.attn_param_shapes(cfg, kind).items():
                s[p + "attn." + n] = shp
        else:
            s[p + "attn.gate_logits"] = (3,)
            s[p + "attn.wq.weight"] = (cfg.n_head * hd, D)
            s[p + "attn.wk.weight"] = (kv, D)
            s[p + "attn.wv.weight"] = (kv, D)
            s[p + "attn.proj.weight"] = (D, cfg.n_head * hd)
            s[p + "attn.global_tokens.weight"] = (cfg.num_global_tokens, D)
        if kind == "mod":
            s[p + "ffn.part_router.gate.weight"] = (cfg.num_dense_parts, D)
            for q in range(cfg.num_dense_parts):
                s[p + f"ffn.parts.{q}.router.gate.weight"] = (cfg.num_experts_per_part, D)
                for e in range(cfg.num_experts_per_part):
                    pe = p + f"ffn.parts.{q}.experts.{e}."
                    s[pe + "w_gate.weight"] = (cfg.expert_hidden, D)
                    s[pe + "w_up.weight"] = (cfg.expert_hidden, D)
                    s[pe + "w_down.weight"] = (D, cfg.expert_hidden)
        else:
            s[p + "ffn.w_gate.weight"] = (cfg.mlp_hidden, D)
            s[p + "ffn.w_up.weight"] = (cfg.mlp_hidden, D)
            s[p + "ffn.w_down.weight"] = (D, cfg.mlp_hidden)
    return s


def init_state_dict(cfg: Config, seed: int, gate_std: float = 0.0) -> dict:
    """Seeded N(0, init_std) weights with the reference's residual scaling
    (cometspark.py:455-481: attn.proj and SwiGLU w_down times 1/sqrt(2*n_layer)),
    unit norm gains and zero gate logits.  Each tensor has its own stream
    (seed, name hash) so large models can be built tensor by tensor."""
    sd = {}
    rs = F32(1.0 / ((2 * cfg.n_layer) ** 0.5))
    for j, (name, shape) in enumerate(param_shapes(cfg).items()):
        if name == "head.weight" and cfg.tie_weights:
            continue
        if name.endswith("norm1.weight") or name.endswith("norm2.weight") or name == "norm.weight":
            sd[name] = np.ones(shape, dtype=F32)
        elif name.endswith("gate_logits"):
            rng = np.random.default_rng([seed, j])
            sd[name] = (rng.standard_normal(shape) * gate_std).astype(F32)
        else:
            rng = np.random.default_rng([seed, j])
            w = rng.standard_normal(shape, dtype=F32) * F32(cfg.init_std)
            if name.endswith("attn.proj.weight") or (name.endswith("ffn.w_down.weight")):
                w = w * rs
            sd[name] = w.astype(F32)
    if cfg.tie_weights:
        sd["head.weight"] = sd["tok_emb.weight"]
    return sd


# ---------------------------------------------------------------------------
# primitives
# ---------------------------------------------------------------------------

def rmsnorm(x, w, eps=1e-6):
    ms = np.mean(x * x, axis=-1, keepdims=True, dtype=F32)
    return (x / np.sqrt(ms + F32(eps)) * w).astype(F32)


def linear(x, W):
    return (x @ W.T).astype(F32)


def silu(x):
    return (x * (F32(0.5) * (F32(1.0) + np.tanh(F32(0.5) * x)))).astype(F32)


def softmax(x):
    m = np.max(x, axis=-1, keepdims=True)
    e = np.exp(x - m)
    return (e / np.sum(e, axis=-1, keepdims=True)).astype(F32)


def rope_table(head_dim, max_seq, theta=10000.0):
    half = head_dim // 2
    i = np.arange(half, dtype=F32)
    inv_freq = 1.0 / (theta ** (2.0 * i / head_dim))
    pos = np.arange(max_seq, dtype=F32)
    ang = np.outer(pos, inv_freq)
    cos = np.concatenate([np.cos(ang), np.cos(ang)], axis=-1)
    sin = np.concatenate([np.sin(ang), np.sin(ang)], axis=-1)
    return cos, sin


def apply_rope(x, pos, cos, sin):
    """x [B,T,H,d]; pos [T] or [B,T] absolute positions."""
    half = x.shape[-1] // 2
    c = cos[pos]
    s = sin[pos]
    if c.ndim == 2:
        c, s = c[None, :, None, :], s[None, :, None, :]
    else:
        c, s = c[:, :, None, :], s[:, :, None, :]
    rot = np.concatenate([-x[..., half:], x[..., :half]], axis=-1)
    return (x * c + rot * s).astype(x.dtype)


def tree_depths_and_ancestors(parents):
    """parents[i] < i is the parent node or -1 for a child of the last
    committed token.  Returns depth [T] and the ancestor-or-self mask [T,T]."""
    T = len(parents)
    depth = np.zeros(T, dtype=np.int64)
    anc = np.zeros((T, T), dtype=bool)
    for i in range(T):
        anc[i, i] = True
        p = int(parents[i])
        if p >= 0:
            if p >= i:
                raise ValueError("parents must be topologically ordered")
            depth[i] = depth[p] + 1
            anc[i] |= anc[p]
    return depth, anc


def attention(sd, cfg: Config, prefix, x, cache, parents, rope, recurrent=False):
    """TriSparseAttention.forward for x [B,T,D] on top of `cache`
    ({'k','v'} each [B,Tc,n_kv,hd], or None).

    recurrent=True restates TriSparseAttention.forward_recurrent (tri_sparse_attn.py:619-760): the state keeps
    only the last `window_size` keys (:676-684), so the ALiBi path sees those keys only and stays switched on
    as long as that count is at most 1024 (:717); the cache kept here is untrimmed and the window is applied
    as a mask, which selects the same keys."""
    B, T, D = x.shape
    H, hd, n_kv = cfg.n_head, cfg.head_dim, cfg.n_kv_head
    n_rep = H // n_kv
    Tc = 0 if cache is None else cache["k"].shape[1]
    if parents is None:
        depth = np.arange(T)
        vis_new = np.tril(np.ones((T, T), dtype=bool))
    else:
        depth, vis_new = tree_depths_and_ancestors(parents)
    pos = Tc + depth  # absolute position of each new token

    wq, wk, wv = (sd[prefix + f"attn.{n}.weight"] for n in ("wq", "wk", "wv"))
    q = linear(x, wq).reshape(B, T, H, hd)
    k = linear(x, wk).reshape(B, T, n_kv, hd)
    v = linear(x, wv).reshape(B, T, n_kv, hd)
    if cfg.use_rope:
        cos, sin = rope
        q = apply_rope(q, pos, cos, sin)
        k = apply_rope(k, pos, cos, sin)
    if cache is not None:
        k_all = np.concatenate([cache["k"], k], axis=1)
        v_all = np.concatenate([cache["v"], v], axis=1)
    else:
        k_all, v_all = k, v
    new_cache = {"k": k_all, "v": v_all}
    Tk = Tc + T
    key_pos = np.concatenate([np.arange(Tc), pos])

    kr = np.repeat(k_all, n_rep, axis=2).transpose(0, 2, 1, 3)  # B,H,Tk,d
    vr = np.repeat(v_all, n_rep, axis=2).transpose(0, 2, 1, 3)
    qh = q.transpose(0, 2, 1, 3)
    scale = F32(1.0 / (hd ** 0.5))
    scores = (qh @ kr.transpose(0, 1, 3, 2)) * scale  # B,H,T,Tk

    visible = np.zeros((T, Tk), dtype=bool)
    visible[:, :Tc] = True
    visible[:, Tc:] = vis_new
    dist = pos[:, None] - key_pos[None, :]
    mask_a = np.where(visible & (dist < cfg.window_size) & (dist >= 0), 0.0, -1e9).astype(F32)
    out_a = softmax(scores + mask_a[None, None]) @ vr

    g = sd[prefix + "attn.global_tokens.weight"]
    n_g = g.shape[0]
    kg = np.repeat(linear(g, wk).reshape(n_g, n_kv, hd), n_rep, axis=1).transpose(1, 0, 2)
    vg = np.repeat(linear(g, wv).reshape(n_g, n_kv, hd), n_rep, axis=1).transpose(1, 0, 2)
    out_b = softmax((qh @ kg.transpose(0, 2, 1)[None]) * scale) @ vg[None]

    gate = (1.0 / (1.0 + np.exp(-sd[prefix + "attn.gate_logits"].astype(F32)))).astype(F32)
    out = gate[0] * out_a + gate[1] * out_b

    if cfg.use_alibi:
        tk_eff = np.full(T, Tk) if parents is None else (pos + 1)
        if recurrent:
            tk_eff = np.minimum(pos + 1, cfg.window_size)
        use_c = tk_eff <= ALIBI_MAX_T
        if np.any(use_c):
            slopes = (1.0 / (2.0 ** (np.arange(1, H + 1, dtype=F32) / H))).astype(F32)
            seen = visible & (dist < cfg.window_size) if recurrent else visible
            bias = np.where(seen & (dist >= 0),
                            -slopes[:, None, None] * dist[None].astype(F32),
                            F32(-1e9)).astype(F32)
            out_c = softmax(scores + bias[None]) @ vr
            out = out + gate[2] * out_c * use_c[None, None, :, None].astype(F32)

    out = out.transpose(0, 2, 1, 3).reshape(B, T, D)
    return linear(out.astype(F32), sd[prefix + "attn.proj.weight"]), new_cache


def swiglu(x, wg, wu, wd):
    return linear(silu(linear(x, wg)) * linear(x, wu), wd)


def route(x, gate_w, top_k):
    """Router.forward at inference: top-k on logits, softmax over the kept logits."""
    logits = linear(x, gate_w)
    idx = np.argsort(-logits, axis=-1, kind="stable")[..., :top_k]
    w = softmax(np.take_along_axis(logits, idx, axis=-1))
    return idx, w


def mod_layer(sd, cfg: Config, prefix, x):
    P, E = cfg.num_dense_parts, cfg.num_experts_per_part
    xf = x.reshape(-1, x.shape[-1])
    pidx, pw = route(xf, sd[prefix + "ffn.part_router.gate.weight"], P)
    part_w = np.zeros((xf.shape[0], P), dtype=F32)
    np.put_along_axis(part_w, pidx, pw, axis=-1)
    out = np.zeros_like(xf)
    for p in range(P):
        pp = prefix + f"ffn.parts.{p}."
        eidx, ew = route(xf, sd[pp + "router.gate.weight"], cfg.top_k)
        comb = np.zeros_like(xf)
        for e in range(E):
            slot = eidx == e
            tok = slot.any(axis=-1)
            if not tok.any():
                continue
            pe = pp + f"experts.{e}."
            y = swiglu(xf[tok], sd[pe + "w_gate.weight"], sd[pe + "w_up.weight"], sd[pe + "w_down.weight"])
            w_e = (ew * slot).sum(axis=-1)[tok]
            comb[tok] += y * w_e[:, None]
        out += comb * part_w[:, p:p + 1]
    return out.reshape(x.shape).astype(F32)


def forward_hidden(sd, cfg: Config, tokens, cache=None, parents=None, recurrent=False):
    """Final-norm hidden states [B,T,D] and the new per-layer KV cache."""
    tokens = np.asarray(tokens, dtype=np.int64)
    x = sd["tok_emb.weight"][tokens].astype(F32)
    if cfg.embedding_scale:
        x = (x * F32(np.sqrt(cfg.dim))).astype(F32)
    Tc = 0 if cache is None else cache_len(cache)
    rope = rope_table(cfg.head_dim, max(cfg.max_seq_len, Tc + tokens.shape[1] + 1),
                      cfg.rope_theta) if cfg.use_rope else None
    new_cache = []
    for i, kind in enumerate(cfg.layer_pattern):
        p = f"blocks.{i}."
        if kind in DELTA_KINDS:
            a, c = delta.attention(sd, cfg, p + "attn.", kind, rmsnorm(x, sd[p + "norm1.weight"]),
                                   None if cache is None else cache[i], parents, rope, recurrent)
        else:
            a, c = attention(sd, cfg, p, rmsnorm(x, sd[p + "norm1.weight"]),
                             None if cache is None else cache[i], parents, rope, recurrent)
        new_cache.append(c)
        x = x + a
        h = rmsnorm(x, sd[p + "norm2.weight"])
        if kind == "mod":
            x = x + mod_layer(sd, cfg, p, h)
        else:
            x = x + swiglu(h, sd[p + "ffn.w_gate.weight"], sd[p + "ffn.w_up.weight"],
                           sd[p + "ffn.w_down.weight"])
    return rmsnorm(x, sd["norm.weight"]), new_cache


def forward(sd, cfg: Config, tokens, cache=None, parents=None, recurrent=False):
    """Logits [B,T,V] and the new cache."""
    h, c = forward_hidden(sd, cfg, tokens, cache, parents, recurrent)
    return linear(h, sd["head.weight"]), c


def generate_greedy_recurrent(sd, cfg: Config, prompt, max_new_tokens, eos_id=None):
    """`generate` with its default arguments (cometspark.py:773-866): greedy decoding on the recurrent path.
    The prompt warms the state up token by token, then the LAST PROMPT TOKEN IS FED A SECOND TIME and its logits
    give the first new token (:848-856); generation stops early when every row emits `eos_id`, and an `eos_id`
    column is appended when the last column is not all `eos_id` (:823-829)."""
    cur = np.asarray(prompt, dtype=np.int64)
    if cur.ndim == 1:
        cur = cur[None, :]
    _, cache = forward(sd, cfg, cur, recurrent=True)       # a causal forward equals token-by-token warm-up
    for _ in range(int(max_new_tokens)):
        lg, cache = forward(sd, cfg, cur[:, -1:], cache=cache, recurrent=True)
        nxt = np.argmax(lg[:, -1], axis=-1).astype(np.int64)
        cur = np.concatenate([cur, nxt[:, None]], axis=1)
        if eos_id is not None and np.all(nxt == eos_id):
            break
    if eos_id is not None and cur.shape[1] > 0 and not np.all(cur[:, -1] == eos_id):
        cur = np.concatenate([cur, np.full((cur.shape[0], 1), eos_id, dtype=cur.dtype)], axis=1)
    return cur


def cache_len(cache):
    """Cached positions per sequence (a vda layer's entry nests one cache per sub-module)."""
    c = cache[0]
    while "k" not in c:
        c = next(iter(c.values()))
    return c["k"].shape[1]


def commit_cache(cache, base_len, keep_slots):
    """KV commit / rollback: keep the first `base_len` cached positions and,
    of the entries appended after them, those at `keep_slots` (in order)."""
    sel = np.concatenate([np.arange(base_len), base_len + np.asarray(keep_slots, dtype=np.int64)])

    def pick(c):
        if "k" in c:
            return {"k": c["k"][:, sel], "v": c["v"][:, sel]}
        return {n: pick(v) for n, v in c.items()}
    return [pick(c) for c in cache]


def bf16_round(a):
    """Round-to-nearest-even float32 -> bfloat16 -> float32."""
    a = np.ascontiguousarray(a, dtype=F32)
    u = a.view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    out = ((u + r) & np.uint32(0xFFFF0000)).astype(np.uint32)
    nan = np.isnan(a)
    if np.any(nan):
        out = np.where(nan, u | np.uint32(0x00400000), out)
    return out.view(F32)
