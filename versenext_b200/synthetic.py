"""Seeded synthetic weights for benchmarks and smoke runs.

Random N(0, init_std) weights of the VerseNexLM architecture with the reference's residual scaling
(verse_nex/cometspark.py:455-481: attn.proj and SwiGLU w_down times 1/sqrt(2 n_layer)), unit norm gains
and zero gate logits.  Tensors are produced one at a time so that a 1.1 B-parameter model never sits on
the host in full.
"""

from __future__ import annotations

from typing import Iterator, Tuple

import numpy as np


def mate_kwargs(**over) -> dict:
    """CometSparkV05 factory defaults (spark/src/base_model.py:760-786)."""
    kw = dict(vocab_size=248320, dim=1024, n_layer=20, n_head=16, n_kv_head=8,
              layer_pattern=["mod" if i % 4 == 0 else "trisparse" for i in range(20)],
              window_size=1024, num_global_tokens=128, use_alibi=False, use_rope=True, max_seq_len=4096,
              num_dense_parts=4, num_experts_per_part=4, top_k=2, tie_weights=True, embedding_scale=True)
    kw.update(over)
    return kw


def draft_kwargs(**over) -> dict:
    """The small draft of the full speculative-decode workload: 2 layers, dim 256, 4 heads, all TriSparse."""
    kw = dict(vocab_size=248320, dim=256, n_layer=2, n_head=4, max_seq_len=2048)
    kw.update(over)
    return kw


def _shapes(kw: dict) -> Iterator[Tuple[str, tuple]]:
    D, H = kw["dim"], kw["n_head"]
    n_kv = kw.get("n_kv_head") or H
    hd = D // H
    pattern = kw.get("layer_pattern") or ["trisparse"] * kw["n_layer"]
    mult = kw.get("mlp_hidden_multiple", 4)
    hidden = int((mult * D * 2 / 3 + 63) // 64) * 64
    eh = kw.get("expert_hidden") or max(int(D * 8 / 3 / 64) * 64, 64)
    P, E = kw.get("num_dense_parts", 5), kw.get("num_experts_per_part", 8)
    yield "tok_emb.weight", (kw["vocab_size"], D)
    yield "norm.weight", (D,)
    if not kw.get("tie_weights", True):
        yield "head.weight", (kw["vocab_size"], D)
    for i, kind in enumerate(pattern):
        p = f"blocks.{i}."
        yield p + "norm1.weight", (D,)
        yield p + "norm2.weight", (D,)
        n_g = kw.get("num_global_tokens", 64)
        if kind in ("vda", "dsa", "kda", "gmla"):
            # the modules of verse_nex/delta_attention.py: a vda layer holds one of each under its own prefix
            lat = kw.get("latent_dim") or n_kv * hd
            for sub in (("dsa", "kda", "gmla") if kind == "vda" else (kind,)):
                q = p + "attn." + (sub + "." if kind == "vda" else "")
                yield q + "wq.weight", (H * hd, D)
                if sub == "gmla":
                    yield q + "w_kv_down.weight", (lat, D)
                    yield q + "w_k_up.weight", (n_kv * hd, lat)
                    yield q + "w_v_up.weight", (n_kv * hd, lat)
                else:
                    yield q + "wk.weight", (n_kv * hd, D)
                    yield q + "wv.weight", (n_kv * hd, D)
                if sub == "dsa":
                    yield q + "global_tokens.weight", (n_g, D)
                if sub != "kda":
                    yield q + "head_gate_logits", (H,)
            if kind == "vda":
                yield p + "attn.gate_logits", (3,)
            yield p + "attn.proj.weight", (D, H * hd)
        else:
            yield p + "attn.gate_logits", (3,)
            yield p + "attn.wq.weight", (H * hd, D)
            yield p + "attn.wk.weight", (n_kv * hd, D)
            yield p + "attn.wv.weight", (n_kv * hd, D)
            yield p + "attn.proj.weight", (D, H * hd)
            yield p + "attn.global_tokens.weight", (n_g, D)
        if kind == "mod":
            yield p + "ffn.part_router.gate.weight", (P, D)
            for q in range(P):
                yield p + f"ffn.parts.{q}.router.gate.weight", (E, D)
                for e in range(E):
                    pe = p + f"ffn.parts.{q}.experts.{e}."
                    yield pe + "w_gate.weight", (eh, D)
                    yield pe + "w_up.weight", (eh, D)
                    yield pe + "w_down.weight", (D, eh)
        else:
            yield p + "ffn.w_gate.weight", (hidden, D)
            yield p + "ffn.w_up.weight", (hidden, D)
            yield p + "ffn.w_down.weight", (D, hidden)


def random_tensors(kw: dict, seed: int, init_std: float = 0.02) -> Iterator[Tuple[str, np.ndarray]]:
    rs = np.float32(1.0 / ((2 * kw["n_layer"]) ** 0.5))
    for j, (name, shape) in enumerate(_shapes(kw)):
        if name.endswith(("norm1.weight", "norm2.weight")) or name == "norm.weight":
            yield name, np.ones(shape, dtype=np.float32)
        elif name.endswith("gate_logits"):
            yield name, np.zeros(shape, dtype=np.float32)
        else:
            rng = np.random.default_rng([seed, j])
            w = rng.standard_normal(shape, dtype=np.float32) * np.float32(init_std)
            if name.endswith("attn.proj.weight") or name.endswith("ffn.w_down.weight"):
                w *= rs
            yield name, w


def load_random(model, kw: dict, seed: int, init_std: float = 0.02):
    """Fill a device model tensor by tensor and finalise it."""
    for name, w in random_tensors(kw, seed, init_std):
        model.load_tensor(name, w)
    model.finalize()
    return model


def param_count(kw: dict) -> int:
    return int(sum(int(np.prod(s)) for _, s in _shapes(kw)))
