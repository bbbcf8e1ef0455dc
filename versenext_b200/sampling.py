"""Acceptance / rejection sampling and plain sampling on the device.

Thin wrappers over `vn_accept` / `vn_accept_strided`.  They replace the
argmax compare of SpeculativeDecoder.verify (verse_nex/speculative.py:218-223),
the accept loop of verify_then_commit (:280-287) and the temperature /
top-k / rng.choice sampling of cometspark.py:892-911.
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from .device import Context, DeviceArray, as_device


def _ptr(a):
    return C.c_void_p(a.ptr) if a is not None else C.c_void_p(None)


def accept(ctx: Context, p_logits, q_logits, draft_tokens, *, u_accept=None, u_sample=None,
           seed: int = 0, offset: int = 0, temperature: float = 1.0, top_k: int = 0,
           bonus: bool = True, p_strides=None, q_strides=None, shape=None, out=None):
    """Run the acceptance rule for a batch.

    p_logits [B, k+1, V] (or [B, k, V] when `bonus` is False) target logits,
    q_logits [B, k, V] draft logits or None, draft_tokens [B, k] int64.
    `p_strides` / `q_strides` = (batch stride, position stride) in elements for
    non-contiguous row layouts; then `shape` = (B, k, V) must be given.
    Returns (accept_len DeviceArray int32 [B], tokens DeviceArray int64 [B, k+1]).
    """
    p = as_device(ctx, p_logits, np.float32)
    q = as_device(ctx, q_logits, np.float32) if q_logits is not None else None
    d = as_device(ctx, draft_tokens, np.int64)
    if shape is None:
        B, k = d.shape
        V = p.shape[-1]
    else:
        B, k, V = shape
    ua = as_device(ctx, u_accept, np.float32) if u_accept is not None else None
    us = as_device(ctx, u_sample, np.float32) if u_sample is not None else None
    if out is None:
        out_len = ctx.empty((B,), np.int32)
        out_tok = ctx.empty((B, k + 1), np.int64)
    else:
        out_len, out_tok = out
    np_rows = k + 1 if bonus else k
    ps = p_strides if p_strides is not None else (np_rows * V, V)
    qs = q_strides if q_strides is not None else (k * V, V)
    ctx._check(ctx.lib.vn_accept_strided(
        ctx.handle, _ptr(p), ps[0], ps[1], _ptr(q), qs[0], qs[1], _ptr(d), _ptr(ua), _ptr(us),
        int(seed) & 0xFFFFFFFFFFFFFFFF, int(offset) & 0xFFFFFFFF, float(temperature), int(top_k or 0),
        int(bool(bonus)), B, k, V, _ptr(out_len), _ptr(out_tok)))
    return out_len, out_tok


def sample(ctx: Context, logits, *, temperature: float = 1.0, top_k: int = 0, seed: int = 0,
           offset: int = 0, uniforms=None) -> DeviceArray:
    """One token per row of logits [R, V]: argmax when temperature <= 0, else
    softmax(logits / T) restricted to the top-k, drawn by inverse CDF."""
    lg = as_device(ctx, logits, np.float32)
    R, V = lg.size // lg.shape[-1], lg.shape[-1]
    empty = ctx.empty((R, 0), np.int64)
    us = None
    ua = None
    if uniforms is not None:
        us = as_device(ctx, np.asarray(uniforms, dtype=np.float32).reshape(R, 1), np.float32)
        ua = ctx.empty((R, 0), np.float32)
    _, tok = accept(ctx, lg, None, empty, u_accept=ua, u_sample=us, seed=seed, offset=offset,
                    temperature=temperature, top_k=top_k, bonus=True, shape=(R, 0, V),
                    p_strides=(V, V), q_strides=(0, 0))
    return tok.reshape(R)


def argmax(ctx: Context, logits) -> DeviceArray:
    return sample(ctx, logits, temperature=0.0)


def philox_uniforms(ctx: Context, seed: int, offset: int, B: int, n: int, purpose: int) -> np.ndarray:
    out = ctx.empty((B, n), np.float32)
    ctx._check(ctx.lib.vn_philox_uniform(ctx.handle, int(seed), int(offset), B, n, purpose, _ptr(out)))
    return out.numpy()
