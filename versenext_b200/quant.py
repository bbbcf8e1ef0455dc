"""Weight-only quantisation on the device: the reference's `quantize_int8` / `quantize_int4`
(verse_torch/quantize.py:187-258) as one kernel call.

`quantize(ctx, w, scheme)` returns `(q, scale)` as device arrays with the reference's layouts:
int8 `(out, in)` or packed uint8 `(out, ceil(in / 2))` (even index in the low nibble, :36-66) and float32
scales `(out, 1)`; `"int4g128"` keeps one bf16-representable scale per 128 input features, `(out, ceil(in / 128))`.
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from .device import Context, as_device

SCHEMES = ("int8", "int4", "int4g128")


def quantize(ctx: Context, w, scheme: str = "int8"):
    if scheme not in SCHEMES:
        raise ValueError(f"unknown scheme {scheme!r}, expected one of {SCHEMES}")
    wd = as_device(ctx, w, np.float32)
    if wd.ndim != 2:
        raise ValueError("quantize takes a 2-D (out_features, in_features) matrix")
    rows, K = wd.shape
    if scheme == "int8":
        q = ctx.empty((rows, K), np.int8)
    else:
        q = ctx.empty((rows, (K + 1) // 2), np.uint8)
    sc = ctx.empty((rows, (K + 127) // 128 if scheme == "int4g128" else 1), np.float32)
    ctx._check(ctx.lib.vn_quantize(ctx.handle, C.c_void_p(wd.ptr), rows, K, scheme.encode(), C.c_void_p(q.ptr),
                                   C.c_void_p(sc.ptr)))
    return q, sc
