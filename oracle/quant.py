"""Weight-only quantisation oracle (test infrastructure, CPU, NumPy).

Per-output-channel INT8 / INT4 restate verse_torch/quantize.py:
  quantize_int8 :187-214  scale = max|w|/127, q = round(w/scale).clip(-127,127)
  quantize_int4 :231-258  scale = max|w|/7,   q = round(w/scale).clip(-8,7)
  _pack_int4    :36-66    two's-complement nibbles, even index in the low nibble
  matmul_int4   :277-309  y = (x @ q.T) * scale
Pinned against the real functions by tests/golden/quant_reference.npz.

Group-128 INT4 with bf16 scales has no counterpart in the reference
("parity unpinned"): the same formulas applied to each run of 128 input
features, the scale rounded to bfloat16 before the division.
"""

from __future__ import annotations

import numpy as np

from .model import bf16_round

F32 = np.float32


def quantize_int8(w):
    w = np.asarray(w, dtype=F32)
    max_abs = np.max(np.abs(w), axis=-1, keepdims=True)
    scale = (np.where(max_abs > 0, max_abs, 1.0) / 127.0).astype(F32)
    q = np.round(w / scale).clip(-127, 127).astype(np.int8)
    return q, scale


def pack_int4(q):
    q = np.asarray(q, dtype=np.int8)
    if q.shape[-1] % 2:
        q = np.concatenate([q, np.zeros(q.shape[:-1] + (1,), dtype=np.int8)], axis=-1)
    lo = q[..., 0::2].astype(np.uint8) & 0x0F
    hi = q[..., 1::2].astype(np.uint8) & 0x0F
    return ((hi << 4) | lo).astype(np.uint8)


def unpack_int4(packed, in_dim):
    lo = (packed & 0x0F).astype(np.int16)
    hi = ((packed >> 4) & 0x0F).astype(np.int16)
    lo = np.where(lo >= 8, lo - 16, lo)
    hi = np.where(hi >= 8, hi - 16, hi)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.int8)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out[..., :in_dim]


def quantize_int4(w):
    w = np.asarray(w, dtype=F32)
    max_abs = np.max(np.abs(w), axis=-1, keepdims=True)
    scale = (np.where(max_abs > 0, max_abs, 1.0) / 7.0).astype(F32)
    q = np.round(w / scale).clip(-8, 7).astype(np.int8)
    return pack_int4(q), scale


def quantize_int4_g128(w, group=128):
    """Returns (packed uint8 [out, in/2], scales float32 (bf16-representable) [out, ceil(in/group)]).
    A last group shorter than `group` (the SwiGLU hidden 2752 = 21.5 groups) takes its scale from the
    features it has."""
    w = np.asarray(w, dtype=F32)
    out_dim, in_dim = w.shape
    pad = (-in_dim) % group
    wp = np.pad(w, ((0, 0), (0, pad))) if pad else w
    g = wp.reshape(out_dim, -1, group)
    max_abs = np.max(np.abs(g), axis=-1, keepdims=True)
    scale = bf16_round((np.where(max_abs > 0, max_abs, 1.0) / 7.0).astype(F32))
    q = np.round(g / scale).clip(-8, 7).astype(np.int8).reshape(out_dim, in_dim + pad)[:, :in_dim]
    return pack_int4(np.ascontiguousarray(q)), scale[..., 0]


def dequant_int8(q, scale):
    return q.astype(F32) * scale


def dequant_int4(packed, scale, in_dim):
    return unpack_int4(packed, in_dim).astype(F32) * scale


def dequant_int4_g128(packed, scales, in_dim, group=128):
    q = unpack_int4(packed, in_dim).astype(F32)
    pad = (-in_dim) % group
    if pad:
        q = np.pad(q, ((0, 0), (0, pad)))
    return (q.reshape(q.shape[0], -1, group) * scales[..., None]).reshape(q.shape[0], in_dim + pad)[:, :in_dim]


def linear_int8(x, q, scale):
    """QuantizedLinear fused form: (x @ q.T) * scale (quantize.py:506-533)."""
    return ((np.asarray(x, F32) @ q.astype(F32).T) * scale.reshape(1, -1)).astype(F32)


def linear_int4(x, packed, scale, in_dim):
    return ((np.asarray(x, F32) @ unpack_int4(packed, in_dim).astype(F32).T) * scale.reshape(1, -1)).astype(F32)


def linear_int4_g128(x, packed, scales, in_dim, group=128):
    return (np.asarray(x, F32) @ dequant_int4_g128(packed, scales, in_dim, group).T).astype(F32)
