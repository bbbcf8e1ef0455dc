"""Speculative-decoding loops (test infrastructure, CPU, NumPy).

`draft_heads`, `verify` and `verify_then_commit` restate
SpeculativeDecoder (verse_nex/speculative.py:110-162, :168-224, :230-310):
k bias-free heads on the last hidden state, one target forward over
[context, draft], argmax compare at positions T_ctx-1 .. T_ctx-2+k, longest
matching prefix plus the target's token at the first miss, no bonus token.
Pinned against the real class by tests/golden/spec_reference.npz.

`generate` composes a separate draft model with the target (the reference
has no such loop; its pieces are the reference forward and the rule above).
"""

from __future__ import annotations

import numpy as np

from . import model as M
from .accept import accept, accept_greedy
from .philox import uniforms_for_call


def draft_heads(hidden, heads):
    """hidden [B,T,D] | [B,D]; heads: list of [V,D].  Returns tokens [B,k] int64, logits list."""
    h = np.asarray(hidden, dtype=np.float32)
    if h.ndim == 3:
        h = h[:, -1, :]
    elif h.ndim == 4:
        h = h.reshape(h.shape[0], -1, h.shape[-1])[:, -1, :]
    elif h.ndim != 2:
        raise ValueError("hidden must have 2, 3 or 4 dims")
    logits = [M.linear(h, w) for w in heads]
    return np.stack([np.argmax(l, axis=-1) for l in logits], axis=1).astype(np.int64), logits


def verify(draft_tokens, model_fn, context_tokens):
    draft = np.asarray(draft_tokens)
    ctx = np.asarray(context_tokens)
    if draft.ndim != 2 or ctx.ndim != 2:
        raise ValueError("draft_tokens / context_tokens must be 2-D")
    if draft.shape[0] != ctx.shape[0]:
        raise ValueError("batch mismatch")
    k, T = draft.shape[1], ctx.shape[1]
    logits = model_fn(np.concatenate([ctx, draft], axis=1).astype(np.int64))
    pred = np.argmax(logits[:, T - 1:T - 1 + k, :], axis=-1)
    return draft == pred, pred


def verify_then_commit(draft_tokens, model_fn, context_tokens):
    draft = np.asarray(draft_tokens)[:1]
    ctx = np.asarray(context_tokens)[:1]
    mask, pred = verify(draft, model_fn, ctx)
    toks, ok = [], True
    for i in range(draft.shape[1]):
        if mask[0, i]:
            toks.append(int(draft[0, i]))
        else:
            toks.append(int(pred[0, i]))
            ok = False
            break
    return toks, ok, np.concatenate([ctx, np.asarray(toks, dtype=np.int64)[None]], axis=1)


def greedy_generate(sd, cfg, prompt, n_new):
    """Plain greedy decoding by full re-forward (cometspark.py:885-893 with temperature <= 0)."""
    cur = np.asarray(prompt, dtype=np.int64)
    margins = []
    for _ in range(n_new):
        lg = M.forward(sd, cfg, cur)[0][:, -1]
        top2 = np.partition(lg, -2, axis=-1)[:, -2:]
        margins.append(top2[:, 1] - top2[:, 0])
        cur = np.concatenate([cur, np.argmax(lg, axis=-1)[:, None]], axis=1)
    return cur, np.stack(margins, axis=1)


def generate(t_sd, t_cfg, d_sd, d_cfg, prompt, k, n_new, temperature=0.0, top_k=0,
             seed=0, bonus=False, max_rounds=None):
    """Speculative decoding with a draft MODEL, one request at a time.

    Returns dict(tokens [B, T+n_new], rounds, proposed, accepted).
    Each round: the draft proposes k tokens autoregressively (greedy at
    temperature 0, else sampling from its softmax with Philox uniforms of
    purpose 2+i), the target scores [last committed, drafts], the acceptance
    rule commits 1..k+1 tokens, and both caches roll back to the committed
    length.
    """
    prompt = np.asarray(prompt, dtype=np.int64)
    B = prompt.shape[0]
    out = []
    stats = dict(rounds=0, proposed=0, accepted=0)
    for b in range(B):
        seq = prompt[b:b + 1].copy()
        target_len = prompt.shape[1] + n_new
        rnd = 0
        while seq.shape[1] < target_len and (max_rounds is None or rnd < max_rounds):
            # --- draft k tokens
            d_seq = seq.copy()
            q_rows = []
            for i in range(k):
                lg = M.forward(d_sd, d_cfg, d_seq)[0][:, -1]
                q_rows.append(lg)
                if temperature <= 0:
                    nxt = np.argmax(lg, axis=-1)
                else:
                    from .accept import softmax64, _inverse_cdf
                    from .philox import uniform
                    u = uniform(seed, rnd, b, i, 2)
                    nxt = np.array([_inverse_cdf(softmax64(lg[0], temperature, top_k), float(u))])
                d_seq = np.concatenate([d_seq, nxt[:, None].astype(np.int64)], axis=1)
            draft = d_seq[:, seq.shape[1]:]
            q_logits = np.stack(q_rows, axis=1)
            # --- verify
            lg = M.forward(t_sd, t_cfg, d_seq)[0]
            T = seq.shape[1]
            p_logits = lg[:, T - 1:T + k]
            if temperature <= 0:
                acc, toks = accept_greedy(p_logits, draft, bonus)
            else:
                ua, us = uniforms_for_call(seed, rnd, B, k)
                acc, toks = accept(p_logits, q_logits, draft, ua[b:b + 1], us[b:b + 1],
                                   temperature, top_k, bonus)
            new = toks[0][toks[0] >= 0]
            seq = np.concatenate([seq, new[None]], axis=1)
            stats["rounds"] += 1
            stats["proposed"] += k
            stats["accepted"] += int(acc[0])
            rnd += 1
        out.append(seq[:, :target_len])
    stats["tokens"] = np.concatenate(out, axis=0) if max_rounds is None else out
    return stats
