"""Acceptance / rejection sampling oracle (test infrastructure, CPU, NumPy).

Greedy rule: restates SpeculativeDecoder.verify + verify_then_commit
(verse_nex/speculative.py:218-223 argmax compare, :280-287 longest matching
prefix then the target's token at the first miss).  Pinned against the real
reference by tests/golden/spec_reference.npz.

Stochastic rule (no counterpart in the reference -- "parity unpinned"):
standard speculative rejection sampling composed from the reference's
sampling primitives:
  * p, q = softmax(logits / max(T, 1e-8))           (cometspark.py:895, :1456-1460)
  * top-k keeps every logit >= the k-th largest      (verse_inference/sampler.py:98-102)
  * accept draft token x_i  iff  u_i * q_i(x_i) < p_i(x_i)
  * first rejection at i: draw from normalise(max(0, p_i - q_i)) by inverse
    CDF over ascending token ids with a second uniform
  * all k accepted: draw the bonus token from p_k the same way
Element-wise exponentials are float32 (as the reference's softmax is); every
sum, normalisation and CDF is float64 so that a different summation order on
the GPU cannot move a decision.
"""

from __future__ import annotations

import numpy as np


def scaled_logits(logits: np.ndarray, temperature: float, top_k: int) -> np.ndarray:
    """float32 `logits / max(T,1e-8)` with everything below the k-th largest set to -inf."""
    x = np.asarray(logits, dtype=np.float32)
    if temperature != 1.0:
        x = (x / np.float32(max(temperature, 1e-8))).astype(np.float32)
    V = x.shape[-1]
    if top_k is not None and 0 < top_k < V:
        kth = np.partition(x, V - top_k, axis=-1)[..., V - top_k][..., None]
        x = np.where(x >= kth, x, np.float32(-np.inf)).astype(np.float32)
    return x


def softmax64(logits: np.ndarray, temperature: float = 1.0, top_k: int = 0) -> np.ndarray:
    """Probabilities as float64: float32 exp(x - max), float64 sum and divide."""
    x = scaled_logits(logits, temperature, top_k)
    m = np.max(x, axis=-1, keepdims=True)
    e = np.exp(x - m).astype(np.float32)
    s = np.sum(e, axis=-1, keepdims=True, dtype=np.float64)
    return e.astype(np.float64) / s


def _inverse_cdf(weights: np.ndarray, u: float) -> int:
    """Smallest token id t with cumsum(weights)[t] > u * total (ascending ids)."""
    c = np.cumsum(weights, dtype=np.float64)
    total = c[-1]
    t = int(np.searchsorted(c, np.float64(u) * total, side="right"))
    if t >= len(c):  # only when total == 0 or u == 1: last token with weight
        nz = np.nonzero(weights > 0.0)[0]
        t = int(nz[-1]) if len(nz) else len(c) - 1
    return t


def accept_greedy(p_logits, draft_tokens, bonus: bool = True):
    """Temperature-0 acceptance.

    p_logits [B, n, V] with n >= k (+1 when `bonus`); draft_tokens [B, k].
    Returns (accept_len int32 [B], tokens int64 [B, k+1] padded with -1).
    """
    p_logits = np.asarray(p_logits)
    draft = np.asarray(draft_tokens)
    B, k = draft.shape
    pred = np.argmax(p_logits, axis=-1)
    acc = np.zeros(B, dtype=np.int32)
    out = np.full((B, k + 1), -1, dtype=np.int64)
    for b in range(B):
        n = 0
        while n < k and draft[b, n] == pred[b, n]:
            out[b, n] = draft[b, n]
            n += 1
        acc[b] = n
        if n < k:
            out[b, n] = pred[b, n]
        elif bonus:
            out[b, k] = pred[b, k]
    return acc, out


def accept_stochastic(p_logits, q_logits, draft_tokens, u_accept, u_sample,
                      temperature: float = 1.0, top_k: int = 0, bonus: bool = True):
    """Rejection-sampling acceptance with injected uniforms.

    p_logits [B, k+1, V] target logits, q_logits [B, k, V] draft logits or
    None (deterministic proposals: q is a point mass on the draft token),
    draft_tokens [B, k], u_accept [B, k], u_sample [B, k+1].
    Returns (accept_len int32 [B], tokens int64 [B, k+1] padded with -1).
    """
    draft = np.asarray(draft_tokens)
    B, k = draft.shape
    acc = np.zeros(B, dtype=np.int32)
    out = np.full((B, k + 1), -1, dtype=np.int64)
    for b in range(B):
        n = 0
        emitted = False
        while n < k:
            x = int(draft[b, n])
            p = softmax64(p_logits[b, n], temperature, top_k)
            if q_logits is None:
                q = np.zeros_like(p)
                q[x] = 1.0
            else:
                q = softmax64(q_logits[b, n], temperature, top_k)
            if np.float64(u_accept[b, n]) * q[x] < p[x]:
                out[b, n] = x
                n += 1
                continue
            r = np.maximum(p - q, 0.0)
            if r.sum() <= 0.0:
                r = p
            out[b, n] = _inverse_cdf(r, float(u_sample[b, n]))
            emitted = True
            break
        acc[b] = n
        if not emitted and bonus:
            p = softmax64(p_logits[b, k], temperature, top_k)
            out[b, k] = _inverse_cdf(p, float(u_sample[b, k]))
    return acc, out


def accept(p_logits, q_logits, draft_tokens, u_accept=None, u_sample=None,
           temperature: float = 1.0, top_k: int = 0, bonus: bool = True):
    """Dispatch on temperature exactly as the CUDA entry point does."""
    if temperature <= 0.0:
        return accept_greedy(p_logits, draft_tokens, bonus)
    return accept_stochastic(p_logits, q_logits, draft_tokens, u_accept, u_sample,
                             temperature, top_k, bonus)


def make_cfg2_inputs(batch=64, k=4, vocab=248320, seed=1234):
    """Synthetic inputs of the isolated acceptance workload: draft logits
    N(0, 2^2), target = draft + N(0, 0.5^2) (last target row independent),
    draft tokens drawn from softmax(q)."""
    rng = np.random.default_rng(seed)
    q = rng.normal(0.0, 2.0, (batch, k, vocab)).astype(np.float32)
    p = np.empty((batch, k + 1, vocab), dtype=np.float32)
    p[:, :k] = q + rng.normal(0.0, 0.5, (batch, k, vocab)).astype(np.float32)
    p[:, k] = rng.normal(0.0, 2.0, (batch, vocab)).astype(np.float32)
    draft = np.empty((batch, k), dtype=np.int64)
    for b in range(batch):
        for i in range(k):
            pr = softmax64(q[b, i])
            draft[b, i] = _inverse_cdf(pr, float(rng.random()))
    return p, q, draft


def tree_accept_stochastic(p_logits, tokens, parent_rows, depth, u_child, u_sample,
                           temperature: float = 1.0, top_k: int = 0):
    """Stochastic acceptance on a verified tree whose children are FIXED proposals (the draft's m best tokens at a
    node, distinct, in order) -- no counterpart in the reference ("parity unpinned"); the rule is rejection sampling
    with point-mass proposals, applied child after child:

      at a row with target distribution p (softmax of logits / T over the top-k set, as in `softmax64`), remaining
      mass R = 1: child c with token x is accepted iff u_child[b, c] * R < p(x); otherwise x leaves the support
      (R -= p(x)) and the next child is tried.  P(first child) = p(x1), P(second) = (1 - p(x1)) * p(x2) / (1 - p(x1))
      = p(x2), ...: every token is committed with exactly its target probability.  When no child is accepted, or the
      row has none, the row's token is drawn from p without the rejected children (inverse CDF over ascending token
      ids with u_sample[b, row]) and the walk ends.

    p_logits [B, T, V]: row 0 = after the last committed token, row r = after node row r; tokens [B, T] (row 0 is
    the last committed token itself); parent_rows [T]: parent row of every row (-1 for row 0); u_child, u_sample
    [B, T].  Returns (accept_len [B], tokens [B, depth + 1] padded with -1, path rows [B, depth + 1] padded with 0)."""
    tokens = np.asarray(tokens)
    B, T = tokens.shape
    acc = np.zeros(B, dtype=np.int32)
    out = np.full((B, depth + 1), -1, dtype=np.int64)
    path = np.zeros((B, depth + 1), dtype=np.int32)
    for b in range(B):
        cur, a = 0, 0
        while True:
            p = softmax64(p_logits[b, cur], temperature, top_k)
            R = np.float64(1.0)
            removed = []
            took = -1
            if a < depth:
                for c in range(cur + 1, T):
                    if parent_rows[c] != cur:
                        continue
                    x = int(tokens[b, c])
                    if np.float64(u_child[b, c]) * R < p[x]:
                        took = c
                        break
                    removed.append(x)
                    R = R - p[x]
            if took >= 0:
                out[b, a] = tokens[b, took]
                a += 1
                path[b, a] = took
                cur = took
                continue
            r = p.copy()
            r[removed] = 0.0
            if r.sum() <= 0.0:
                r = p
            out[b, a] = _inverse_cdf(r, float(u_sample[b, cur]))
            break
        acc[b] = a
    return acc, out, path
