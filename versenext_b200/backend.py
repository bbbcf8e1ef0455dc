"""`DeviceBackend("cuda")` plugin: the reference's operator set on B200.

Mirrors verse_torch/device.py:219-270 (the abstract operator set),
:285-335 (NumPy semantics each operator must reproduce) and :346-389
(`get_backend` cached factory, `clear_backend_cache`).  Every operator takes
host ndarrays or `DeviceArray`s and returns a `DeviceArray` (the
"backend-native array" of this backend); `np.asarray(result)` copies it back.
All arithmetic is float32 and runs in libvn_b200.so -- there is no host
implementation behind these methods.
"""

from __future__ import annotations

import abc
import ctypes as C

import numpy as np

from .device import Context, DeviceArray, as_device


class DeviceBackend(abc.ABC):
    """Same abstract surface as the reference's DeviceBackend (device.py:219-270)."""

    @property
    @abc.abstractmethod
    def device_type(self) -> str: ...

    @abc.abstractmethod
    def matmul(self, a, b): ...

    @abc.abstractmethod
    def linear(self, x, weight, bias=None): ...

    @abc.abstractmethod
    def softmax(self, x, dim: int = -1): ...

    @abc.abstractmethod
    def layernorm(self, x, weight, bias, eps: float = 1e-5): ...

    @abc.abstractmethod
    def rmsnorm(self, x, weight, eps: float = 1e-6): ...

    @abc.abstractmethod
    def rope(self, x, cos=None, sin=None): ...

    @abc.abstractmethod
    def attention(self, q, k, v, mask=None): ...


def _parse_index(device) -> int:
    s = str(device).lower()
    if s in ("cuda", "gpu"):
        return 0
    if s.startswith("cuda:"):
        return int(s.split(":", 1)[1])
    raise RuntimeError(f"versenext_b200 only provides the 'cuda' backend, got device {device!r}")


def _p(a):
    return C.c_void_p(a.ptr if a is not None else None)


class B200Backend(DeviceBackend):
    def __init__(self, device="cuda"):
        self.device = str(device).lower()
        self.ctx = Context.get(_parse_index(self.device))

    @property
    def device_type(self) -> str:
        return "cuda"

    def _f32(self, x) -> DeviceArray:
        return as_device(self.ctx, x, np.float32)

    def to_device(self, x, dtype=None) -> DeviceArray:
        return as_device(self.ctx, x, dtype)

    # -- operators -----------------------------------------------------------
    def matmul(self, a, b):
        a, b = self._f32(a), self._f32(b)
        if a.ndim < 2 or b.ndim < 2:
            raise ValueError("matmul needs at least 2-D operands")
        M, K = a.shape[-2:]
        K2, N = b.shape[-2:]
        if K != K2:
            raise ValueError(f"matmul: inner dimensions differ ({K} vs {K2})")
        lead = a.shape[:-2]
        batch = int(np.prod(lead, dtype=np.int64))
        if b.ndim == 2:
            bcast = 1
        elif b.shape[:-2] == lead:
            bcast = 0
        else:  # general broadcasting: materialise on the host (rare, small)
            full = np.broadcast_shapes(lead, b.shape[:-2])
            a = self._f32(np.broadcast_to(a.numpy(), full + (M, K)))
            b = self._f32(np.broadcast_to(b.numpy(), full + (K, N)))
            lead, batch, bcast = full, int(np.prod(full, dtype=np.int64)), 0
        out = self.ctx.empty(lead + (M, N), np.float32)
        self.ctx._check(self.ctx.lib.vn_matmul(self.ctx.handle, _p(a), _p(b), _p(out), batch, M, N, K, bcast))
        return out

    def linear(self, x, weight, bias=None):
        x, w = self._f32(x), self._f32(weight)
        b = self._f32(bias) if bias is not None else None
        N, K = w.shape
        if x.shape[-1] != K:
            raise ValueError(f"linear: x has {x.shape[-1]} features, weight expects {K}")
        M = x.size // K if K else 0
        out = self.ctx.empty(x.shape[:-1] + (N,), np.float32)
        self.ctx._check(self.ctx.lib.vn_linear(self.ctx.handle, _p(x), _p(w), _p(b), _p(out), M, N, K))
        return out

    def softmax(self, x, dim: int = -1):
        x = self._f32(x)
        d = dim % x.ndim
        outer = int(np.prod(x.shape[:d], dtype=np.int64))
        inner = int(np.prod(x.shape[d + 1:], dtype=np.int64))
        out = self.ctx.empty(x.shape, np.float32)
        self.ctx._check(self.ctx.lib.vn_softmax(self.ctx.handle, _p(x), _p(out), outer, x.shape[d], inner))
        return out

    def layernorm(self, x, weight, bias, eps: float = 1e-5):
        x, w = self._f32(x), self._f32(weight)
        b = self._f32(bias) if bias is not None else None
        cols = x.shape[-1]
        out = self.ctx.empty(x.shape, np.float32)
        self.ctx._check(self.ctx.lib.vn_layernorm(self.ctx.handle, _p(x), _p(w), _p(b), _p(out),
                                                  x.size // cols, cols, float(eps)))
        return out

    def rmsnorm(self, x, weight, eps: float = 1e-6):
        x, w = self._f32(x), self._f32(weight)
        cols = x.shape[-1]
        out = self.ctx.empty(x.shape, np.float32)
        self.ctx._check(self.ctx.lib.vn_rmsnorm(self.ctx.handle, _p(x), _p(w), _p(out), x.size // cols, cols,
                                                float(eps)))
        return out

    def rope(self, x, cos=None, sin=None):
        if cos is None or sin is None:
            return x  # placeholder behaviour of the reference (device.py:321-323)
        x = self._f32(x)
        D = x.shape[-1]
        half = D // 2
        cos = np.asarray(cos, dtype=np.float32)
        sin = np.asarray(sin, dtype=np.float32)
        # full-D tables carry the half table twice; both forms reduce to (T, half)
        cos = cos[..., :half] if cos.shape[-1] >= D else cos
        sin = sin[..., :half] if sin.shape[-1] >= D else sin
        T = x.shape[-2] if x.ndim >= 2 else 1
        if cos.ndim <= 2 and sin.ndim <= 2:
            # one (T, half) table shared by every leading index of x
            cos, sin = np.broadcast_to(cos, (T, half)), np.broadcast_to(sin, (T, half))
            outer = x.size // (T * D)
        else:
            # tables with leading axes of their own (e.g. one per batch row) broadcast against x[..., :half]
            # exactly as the NumPy expression of the reference does: one table row per row of x
            lead = tuple(x.shape[:-1])
            cos = np.broadcast_to(cos, lead + (half,)).reshape(-1, half)
            sin = np.broadcast_to(sin, lead + (half,)).reshape(-1, half)
            outer, T = 1, x.size // D
        c, s_ = self._f32(np.ascontiguousarray(cos)), self._f32(np.ascontiguousarray(sin))
        out = self.ctx.empty(x.shape, np.float32)
        self.ctx._check(self.ctx.lib.vn_rope(self.ctx.handle, _p(x), _p(c), _p(s_), _p(out), outer, T, D))
        return out

    def attention(self, q, k, v, mask=None):
        q, k, v = self._f32(q), self._f32(k), self._f32(v)
        Tq, D = q.shape[-2:]
        Tk = k.shape[-2]
        if k.shape != v.shape or k.shape[:-2] != q.shape[:-2] or k.shape[-1] != D:
            raise ValueError("attention: q, k, v shapes do not agree")
        m = None
        if mask is not None:
            m = self._f32(np.ascontiguousarray(np.broadcast_to(np.asarray(mask, dtype=np.float32), (Tq, Tk))))
        BH = q.size // (Tq * D)
        out = self.ctx.empty(q.shape, np.float32)
        self.ctx._check(self.ctx.lib.vn_attention(self.ctx.handle, _p(q), _p(k), _p(v), _p(m), _p(out),
                                                  BH, Tq, Tk, D))
        return out


_BACKEND_CACHE: dict = {}


def get_backend(device="cuda") -> DeviceBackend:
    """Cached factory keyed by the lower-cased device string (device.py:381-386)."""
    key = str(device).lower()
    if key not in _BACKEND_CACHE:
        _BACKEND_CACHE[key] = B200Backend(key)
    return _BACKEND_CACHE[key]


def clear_backend_cache() -> None:
    _BACKEND_CACHE.clear()
