"""Device context and NumPy-compatible device buffers on top of the C ABI.

`Context` wraps one `vn_ctx` (one GPU, one stream).  `DeviceArray` is a
contiguous, C-ordered buffer in that GPU's memory with NumPy's `shape` /
`dtype` vocabulary, `__cuda_array_interface__` for zero-copy hand-off, and
`.numpy()` / `np.asarray()` for an explicit device-to-host copy.  It plays the
role that `torch.Tensor` plays for the reference's GPU path
(verse_torch/tensor.py:394 `Tensor.to`, :536-572 `_torch_apply`).
"""

from __future__ import annotations

import ctypes as C
import threading

import numpy as np

from . import _lib


class Event:
    def __init__(self, ctx):
        self.ctx = ctx
        h = C.c_void_p()
        ctx._check(ctx.lib.vn_event_create(ctx.handle, C.byref(h)))
        self.handle = h

    def record(self):
        self.ctx._check(self.ctx.lib.vn_event_record(self.ctx.handle, self.handle))
        return self

    def elapsed_ms(self, later: "Event") -> float:
        ms = C.c_float()
        self.ctx._check(self.ctx.lib.vn_event_elapsed_ms(self.ctx.handle, self.handle, later.handle, C.byref(ms)))
        return float(ms.value)

    def __del__(self):
        try:
            if self.handle:
                self.ctx.lib.vn_event_destroy(self.ctx.handle, self.handle)
        except Exception:
            pass


class Context:
    """One per GPU; cached by device index."""

    _cache: dict = {}
    _lock = threading.Lock()

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        self.device = int(device)
        h = C.c_void_p()
        _lib.check(None, self.lib.vn_ctx_create(self.device, C.byref(h)))
        self.handle = h
        self._pool: dict = {}
        self._pool_class: dict = {}
        self._pool_bytes = 0
        self._pool_lock = threading.Lock()

    @classmethod
    def get(cls, device: int = 0) -> "Context":
        with cls._lock:
            if device not in cls._cache:
                cls._cache[device] = Context(device)
            return cls._cache[device]

    def _check(self, status):
        _lib.check(self.handle, status)

    # -- memory ------------------------------------------------------------
    # Blocks of up to POOL_BLOCK_MAX bytes are kept in size classes when they are freed and handed out again
    # (cudaMalloc / cudaFree cost tens of microseconds each and cudaFree waits for the device).  Everything the
    # context does runs on its one stream, so a block that is reused is touched in stream order.
    POOL_BLOCK_MAX = 64 << 20
    POOL_TOTAL_MAX = 1 << 30

    @staticmethod
    def _size_class(nbytes: int) -> int:
        n = max(int(nbytes), 256)
        if n <= (1 << 20):
            return 1 << (n - 1).bit_length()          # powers of two up to 1 MiB
        return (n + (1 << 20) - 1) & ~((1 << 20) - 1)  # then whole MiB

    def _raw_alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self._check(self.lib.vn_alloc(self.handle, int(nbytes), C.byref(p)))
        return p.value

    def alloc(self, nbytes: int) -> int:
        if nbytes > self.POOL_BLOCK_MAX:
            return self._raw_alloc(nbytes)
        cls = self._size_class(nbytes)
        with self._pool_lock:
            free = self._pool.get(cls)
            if free:
                self._pool_bytes -= cls
                return free.pop()
        try:
            ptr = self._raw_alloc(cls)
        except (MemoryError, RuntimeError):
            self.release_pool()                        # out of memory: give the cached blocks back and try once more
            ptr = self._raw_alloc(cls)
        with self._pool_lock:
            self._pool_class[ptr] = cls
        return ptr

    def free(self, ptr: int):
        with self._pool_lock:
            cls = self._pool_class.get(ptr)
            if cls is not None and self._pool_bytes + cls <= self.POOL_TOTAL_MAX:
                self._pool.setdefault(cls, []).append(ptr)
                self._pool_bytes += cls
                return
            self._pool_class.pop(ptr, None)
        self._check(self.lib.vn_free(self.handle, C.c_void_p(ptr)))

    def release_pool(self):
        """Return every cached block to the driver."""
        with self._pool_lock:
            blocks = [p for lst in self._pool.values() for p in lst]
            self._pool.clear()
            self._pool_bytes = 0
            for p in blocks:
                self._pool_class.pop(p, None)
        for p in blocks:
            self.lib.vn_free(self.handle, C.c_void_p(p))

    def empty(self, shape, dtype=np.float32) -> "DeviceArray":
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        dtype = np.dtype(dtype)
        n = int(np.prod(shape, dtype=np.int64)) * dtype.itemsize
        return DeviceArray(self, self.alloc(n), shape, dtype, owner=True)

    def zeros(self, shape, dtype=np.float32) -> "DeviceArray":
        a = self.empty(shape, dtype)
        if a.nbytes:
            self._check(self.lib.vn_memset(self.handle, C.c_void_p(a.ptr), 0, a.nbytes))
        return a

    def from_numpy(self, arr) -> "DeviceArray":
        arr = np.ascontiguousarray(arr)
        a = self.empty(arr.shape, arr.dtype)
        a.copy_from_host(arr)
        return a

    def pinned(self, shape, dtype=np.float32) -> np.ndarray:
        """Page-locked host array (freed with the process)."""
        dtype = np.dtype(dtype)
        n = int(np.prod(shape, dtype=np.int64)) * dtype.itemsize
        p = C.c_void_p()
        self._check(self.lib.vn_host_alloc(self.handle, max(n, 16), C.byref(p)))
        buf = (C.c_byte * max(n, 16)).from_address(p.value)
        return np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape, dtype=np.int64))).reshape(shape)

    def sync(self):
        self._check(self.lib.vn_sync(self.handle))

    def launch_count(self) -> int:
        n = C.c_uint64()
        self._check(self.lib.vn_launch_count(self.handle, C.byref(n)))
        return int(n.value)

    def flush_l2(self):
        self._check(self.lib.vn_flush_l2(self.handle))

    def profile(self, enable: bool):
        """Bracket every kernel launch with CUDA events (see `profile_report`)."""
        self._check(self.lib.vn_profile(self.handle, int(bool(enable))))

    def profile_report(self) -> dict:
        import json
        buf = C.create_string_buffer(1 << 16)
        self._check(self.lib.vn_profile_report(self.handle, buf, len(buf)))
        return json.loads(buf.value.decode())

    def event(self) -> Event:
        return Event(self)

    def mem_info(self):
        f, t = C.c_size_t(), C.c_size_t()
        self._check(self.lib.vn_mem_info(self.handle, C.byref(f), C.byref(t)))
        return int(f.value), int(t.value)


class DeviceArray:
    """Contiguous C-ordered array in GPU memory."""

    __array_priority__ = 100

    def __init__(self, ctx: Context, ptr: int, shape, dtype, owner=False, base=None):
        self.ctx = ctx
        self.ptr = int(ptr) if ptr else 0
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self._owner = owner
        self._base = base  # keeps the owning buffer alive for views

    @property
    def ndim(self):
        return len(self.shape)

    @property
    def data(self):
        """The array itself: callers written against verse_torch.Tensor read `.data` (tensor.py:394), and a
        device buffer is its own backend-native payload."""
        return self

    @property
    def size(self):
        return int(np.prod(self.shape, dtype=np.int64))

    @property
    def nbytes(self):
        return self.size * self.dtype.itemsize

    @property
    def __cuda_array_interface__(self):
        return {"shape": self.shape, "typestr": self.dtype.str, "data": (self.ptr, False),
                "version": 3, "strides": None}

    def numpy(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=self.dtype)
        if self.nbytes:
            self.ctx._check(self.ctx.lib.vn_d2h(self.ctx.handle, out.ctypes.data_as(C.c_void_p),
                                                C.c_void_p(self.ptr), self.nbytes))
        return out

    def __array__(self, dtype=None, copy=None):
        a = self.numpy()
        return a.astype(dtype) if dtype is not None else a

    def copy_from_host(self, arr):
        arr = np.ascontiguousarray(arr, dtype=self.dtype)
        if arr.size != self.size:
            raise ValueError(f"size mismatch: host {arr.shape} vs device {self.shape}")
        if self.nbytes:
            self.ctx._check(self.ctx.lib.vn_h2d(self.ctx.handle, C.c_void_p(self.ptr),
                                                arr.ctypes.data_as(C.c_void_p), self.nbytes))
        return self

    def copy_from_pinned_async(self, arr: np.ndarray):
        self.ctx._check(self.ctx.lib.vn_h2d_async(self.ctx.handle, C.c_void_p(self.ptr),
                                                  arr.ctypes.data_as(C.c_void_p), self.nbytes))
        return self

    def copy_to_pinned_async(self, arr: np.ndarray):
        self.ctx._check(self.ctx.lib.vn_d2h_async(self.ctx.handle, arr.ctypes.data_as(C.c_void_p),
                                                  C.c_void_p(self.ptr), self.nbytes))
        return arr

    def reshape(self, *shape) -> "DeviceArray":
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = list(shape)
        if -1 in shape:
            known = int(np.prod([s for s in shape if s != -1], dtype=np.int64))
            shape[shape.index(-1)] = self.size // max(known, 1)
        if int(np.prod(shape, dtype=np.int64)) != self.size:
            raise ValueError(f"cannot reshape {self.shape} to {tuple(shape)}")
        return DeviceArray(self.ctx, self.ptr, shape, self.dtype, owner=False, base=self)

    def __getitem__(self, idx) -> "DeviceArray":
        """Views along the leading axis only (int or contiguous slice)."""
        if isinstance(idx, int):
            if idx < 0:
                idx += self.shape[0]
            if not 0 <= idx < self.shape[0]:
                raise IndexError(idx)
            step = self.nbytes // max(self.shape[0], 1)
            return DeviceArray(self.ctx, self.ptr + idx * step, self.shape[1:], self.dtype, base=self)
        if isinstance(idx, slice):
            start, stop, stride = idx.indices(self.shape[0])
            if stride != 1:
                raise IndexError("only contiguous slices are views")
            step = self.nbytes // max(self.shape[0], 1)
            return DeviceArray(self.ctx, self.ptr + start * step, (max(stop - start, 0),) + self.shape[1:],
                               self.dtype, base=self)
        raise IndexError("DeviceArray supports int / slice on the first axis; use .numpy() for the rest")

    def __len__(self):
        return self.shape[0]

    def __repr__(self):
        return f"DeviceArray(shape={self.shape}, dtype={self.dtype}, device=cuda:{self.ctx.device})"

    def __del__(self):
        if getattr(self, "_owner", False) and self.ptr:
            try:
                self.ctx.free(self.ptr)
            except Exception:
                pass
            self.ptr = 0


def as_device(ctx: Context, x, dtype=None) -> DeviceArray:
    """Host ndarray / list -> new device buffer; DeviceArray passes through."""
    if isinstance(x, DeviceArray):
        if dtype is not None and x.dtype != np.dtype(dtype):
            raise TypeError(f"device array has dtype {x.dtype}, need {np.dtype(dtype)}")
        return x
    if hasattr(x, "data") and not isinstance(x, np.ndarray) and hasattr(x, "shape") and hasattr(x, "requires_grad"):
        x = x.data  # reference-style Tensor wrapper
    arr = np.asarray(x)
    if dtype is not None:
        arr = arr.astype(dtype, copy=False)
    return ctx.from_numpy(arr)
