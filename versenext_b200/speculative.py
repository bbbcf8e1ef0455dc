"""`SpeculativeDecoder` with the reference's API, computed on B200.

Same constructor, attributes, methods, return types and exceptions as
verse_nex/speculative.py:55-348:

  * `SpeculativeDecoder(dim, vocab_size, num_draft_heads=4, shared_embedding=None)`
  * `.draft_heads[i].weight.data` is a writable (V, D) float32 array
  * `.draft(hidden)`            -> (tokens (B,k) int64 ndarray, list of k (B,V) logits)
  * `.verify(draft, model, ctx)`-> (accepted_mask (B,k) bool, main_pred (B,k) int64)
  * `.verify_then_commit(...)`  -> (list[int], all_accepted, new_ctx (1, T+n)); row 0 only

`main_model` may be any callable `tokens (B,T) -> logits (B,T,V)` (or a
`(logits, hidden)` tuple): its logits are uploaded and every argmax / compare
runs in the acceptance kernel.  When it is a `versenext_b200.model.VerseNexLM`
the forward itself runs on the device as well.

Additive extensions (defaults reproduce the reference): `temperature`,
`top_k`, `seed`, `bonus` and `draft_logits` on `verify_then_commit` switch on
rejection sampling; `commit_batch` returns every row instead of row 0.
"""

from __future__ import annotations

from typing import Callable, List, Optional, Tuple, Union

import numpy as np

from . import sampling
from .device import Context, DeviceArray, as_device


class Tensor:
    """Minimal stand-in for verse_torch.Tensor at this boundary: `.data`, `.shape`, `.ndim`."""

    requires_grad = False
    grad = None

    def __init__(self, data, requires_grad: bool = False):
        self.data = data

    @property
    def shape(self):
        return tuple(self.data.shape)

    @property
    def ndim(self):
        return len(self.data.shape)


class _Tracked(np.ndarray):
    """ndarray that remembers being written to, so the device copy can be refreshed."""

    def __new__(cls, arr):
        obj = np.asarray(arr).view(cls)
        obj._dirty = [True]
        return obj

    def __array_finalize__(self, obj):
        self._dirty = getattr(obj, "_dirty", [True])

    def __setitem__(self, key, value):
        self._dirty[0] = True
        super().__setitem__(key, value)

    def __array_ufunc__(self, ufunc, method, *inputs, out=None, **kwargs):
        # in-place arithmetic (`w *= 2`, `np.add(w, 1, out=w)`) reaches the array here, not through __setitem__
        plain = tuple(x.view(np.ndarray) if isinstance(x, _Tracked) else x for x in inputs)
        if method == "at" and isinstance(inputs[0], _Tracked):
            inputs[0]._dirty[0] = True
        if out is not None:
            for o in out:
                if isinstance(o, _Tracked):
                    o._dirty[0] = True
            kwargs["out"] = tuple(o.view(np.ndarray) if isinstance(o, _Tracked) else o for o in out)
        res = getattr(ufunc, method)(*plain, **kwargs)
        if out is not None and method != "at":
            return out[0] if len(out) == 1 else out
        return res


class _Param:
    grad = None

    def __init__(self, arr):
        self._data = _Tracked(np.ascontiguousarray(arr, dtype=np.float32))

    @property
    def data(self):
        return self._data

    @data.setter
    def data(self, value):
        self._data = _Tracked(np.ascontiguousarray(value, dtype=np.float32))

    @property
    def shape(self):
        return self._data.shape


class DraftHead:
    """Bias-free Linear(dim, vocab): `.weight.data` (V, D) (speculative.py:101-104)."""

    def __init__(self, dim, vocab, rng):
        bound = 1.0 / np.sqrt(dim)  # kaiming-uniform(a=sqrt 5) bound of the reference Linear (vnnn.py:403-411)
        self.in_features, self.out_features = dim, vocab
        self.weight = _Param(rng.uniform(-bound, bound, (vocab, dim)))
        self.bias = None


def _unwrap(x):
    return x.data if hasattr(x, "data") and not isinstance(x, (np.ndarray, DeviceArray)) else x


class SpeculativeDecoder:
    def __init__(self, dim: int, vocab_size: int, num_draft_heads: int = 4,
                 shared_embedding=None, device: str = "cuda", seed: Optional[int] = None):
        if num_draft_heads < 1:
            raise ValueError(f"num_draft_heads must be >= 1, got {num_draft_heads}")
        self.dim = int(dim)
        self.vocab_size = int(vocab_size)
        self.num_draft_heads = int(num_draft_heads)
        self.shared_embedding = shared_embedding
        rng = np.random.default_rng(seed)
        self.draft_heads = [DraftHead(self.dim, self.vocab_size, rng) for _ in range(self.num_draft_heads)]
        self._device = device
        self._ctx: Optional[Context] = None
        self._w_dev: Optional[DeviceArray] = None
        self._w_ids = [None] * self.num_draft_heads

    # -- device state --------------------------------------------------------
    @property
    def ctx(self) -> Context:
        if self._ctx is None:
            from .backend import _parse_index
            self._ctx = Context.get(_parse_index(self._device))
        return self._ctx

    def _weights(self) -> DeviceArray:
        """Stacked (k*V, D) device copy of the head weights, refreshed when a head changed.

        `head.weight` may be this module's parameter object or anything a caller assigned in its place that
        carries a `.data` array (the reference's tests assign `head.weight = Tensor(ndarray)`,
        tests/test_speculative_decode.py:159-167).  Writes through the tracked array type are seen; a plain
        ndarray cannot report in-place writes, so a head holding one is uploaded again on every call."""
        arrays, dirty = [], self._w_dev is None
        for i, h in enumerate(self.draft_heads):
            w = h.weight
            a = w.data if hasattr(w, "data") and not isinstance(w, np.ndarray) else w
            flag = getattr(a, "_dirty", None)
            if flag is None or flag[0] or self._w_ids[i] != id(a):
                dirty = True
            arrays.append(a)
        if dirty:
            for a in arrays:
                if tuple(np.shape(a)) != (self.vocab_size, self.dim):
                    raise ValueError(f"draft head weight has shape {tuple(np.shape(a))}, "
                                     f"expected {(self.vocab_size, self.dim)}")
            stacked = np.concatenate([np.asarray(a, dtype=np.float32) for a in arrays], axis=0)  # (k*V, D)
            self._w_dev = self.ctx.from_numpy(stacked)
            for i, a in enumerate(arrays):
                self._w_ids[i] = id(a)
                flag = getattr(a, "_dirty", None)
                if flag is not None:
                    flag[0] = False
        return self._w_dev

    # -- draft ---------------------------------------------------------------
    def draft(self, hidden, last_position: Optional[int] = None) -> Tuple[np.ndarray, List[DeviceArray]]:
        h = _unwrap(hidden)
        shape = tuple(h.shape)
        if len(shape) not in (2, 3, 4):
            raise ValueError(f"hidden has {len(shape)} dims, expected 2, 3 or 4")
        if not isinstance(h, DeviceArray):
            h = np.asarray(h, dtype=np.float32)
            if h.ndim == 3:
                h = h[:, -1, :]
            elif h.ndim == 4:  # (B, H, T, D): flatten to (B, -1, D) and take the last row, as the reference does
                h = h.reshape(h.shape[0], -1, h.shape[-1])[:, -1, :]
            h = self.ctx.from_numpy(h)
        else:
            if h.ndim == 3:
                h = _last_rows(self.ctx, h)
            elif h.ndim == 4:
                h = _last_rows(self.ctx, h.reshape(h.shape[0], -1, h.shape[-1]))
        B = h.shape[0]
        k, V, D = self.num_draft_heads, self.vocab_size, self.dim
        if h.shape[1] != D:
            raise ValueError(f"hidden feature size {h.shape[1]} != dim {D}")
        self._last_hidden = h          # (B, D) device rows: what draft_loss(...).backward() differentiates against
        ctx = self.ctx
        logits = ctx.empty((B, k * V), np.float32)   # row b = [head0 | head1 | ...]
        import ctypes as C
        ctx._check(ctx.lib.vn_linear(ctx.handle, C.c_void_p(h.ptr), C.c_void_p(self._weights().ptr), None,
                                     C.c_void_p(logits.ptr), B, k * V, D))
        tokens = sampling.argmax(ctx, logits.reshape(B * k, V)).numpy().reshape(B, k).astype(np.int64)
        per_head = _split_heads(ctx, logits, B, k, V)
        return tokens, per_head

    # -- verify --------------------------------------------------------------
    def _target_logits(self, main_model, full_tokens: np.ndarray):
        out = main_model(Tensor(full_tokens.astype(np.int64)))
        if isinstance(out, tuple):
            out = out[0]
        return as_device(self.ctx, _unwrap(out), np.float32)

    def verify(self, draft_tokens, main_model: Callable, context_tokens) -> Tuple[np.ndarray, np.ndarray]:
        draft = np.asarray(_unwrap(draft_tokens))
        ctx_tok = np.asarray(_unwrap(context_tokens))
        if draft.ndim != 2 or ctx_tok.ndim != 2:
            raise ValueError("draft_tokens / context_tokens must be 2-D (B, k) / (B, T_ctx)")
        if draft.shape[0] != ctx_tok.shape[0]:
            raise ValueError(f"batch mismatch: draft {draft.shape[0]} vs context {ctx_tok.shape[0]}")
        B, k = draft.shape
        T_ctx = ctx_tok.shape[1]
        full = np.concatenate([ctx_tok, draft], axis=1)
        logits = self._target_logits(main_model, full)           # (B, T_ctx + k, V)
        T, V = logits.shape[1], logits.shape[2]
        rows = logits.reshape(B * T, V)[0:B * T]
        # argmax of rows T_ctx-1 .. T_ctx-2+k of every sequence
        pred = np.empty((B, k), dtype=np.int64)
        for b in range(B):
            lo = b * T + T_ctx - 1
            pred[b] = sampling.argmax(self.ctx, rows[lo:lo + k]).numpy()
        return draft == pred, pred

    def verify_then_commit(self, draft_tokens, main_model: Callable, context_tokens,
                           max_redraft_rounds: int = 1, *, temperature: float = 0.0, top_k: int = 0,
                           seed: int = 0, offset: int = 0, bonus: bool = False, draft_logits=None,
                           u_accept=None, u_sample=None):
        draft = np.asarray(_unwrap(draft_tokens))
        ctx_tok = np.asarray(_unwrap(context_tokens))
        toks, lens, new_ctx = self._commit(draft[:1], main_model, ctx_tok[:1], temperature, top_k, seed, offset,
                                           bonus, None if draft_logits is None else draft_logits,
                                           u_accept, u_sample, rows=1)
        k = draft.shape[1]
        accepted = [int(t) for t in toks[0] if t >= 0]
        all_ok = bool(lens[0] == k)
        new_ctx_b = np.concatenate([ctx_tok[:1], np.asarray(accepted, dtype=np.int64)[None, :]], axis=1)
        if not all_ok and max_redraft_rounds > 0:
            # the reference runs one more forward and a draft whose result is discarded (speculative.py:297-308)
            out = main_model(Tensor(new_ctx_b.astype(np.int64)))
            if isinstance(out, tuple):
                out = out[1] if len(out) > 1 else out[0]
            _ = self.draft(out)
        return accepted, all_ok, new_ctx_b

    def commit_batch(self, draft_tokens, main_model: Callable, context_tokens, **kw):
        """Every row's committed tokens: (tokens (B, k+1) padded with -1, accept_len (B,))."""
        draft = np.asarray(_unwrap(draft_tokens))
        ctx_tok = np.asarray(_unwrap(context_tokens))
        toks, lens, _ = self._commit(draft, main_model, ctx_tok, kw.get("temperature", 0.0), kw.get("top_k", 0),
                                     kw.get("seed", 0), kw.get("offset", 0), kw.get("bonus", False),
                                     kw.get("draft_logits"), kw.get("u_accept"), kw.get("u_sample"),
                                     rows=draft.shape[0])
        return toks, lens

    def _commit(self, draft, main_model, ctx_tok, temperature, top_k, seed, offset, bonus, draft_logits,
                u_accept, u_sample, rows):
        if draft.ndim != 2 or ctx_tok.ndim != 2:
            raise ValueError("draft_tokens / context_tokens must be 2-D (B, k) / (B, T_ctx)")
        if draft.shape[0] != ctx_tok.shape[0]:
            raise ValueError(f"batch mismatch: draft {draft.shape[0]} vs context {ctx_tok.shape[0]}")
        B, k = draft.shape
        T_ctx = ctx_tok.shape[1]
        full = np.concatenate([ctx_tok, draft], axis=1)
        logits = self._target_logits(main_model, full)
        T, V = logits.shape[1], logits.shape[2]
        start = logits.reshape(B * T, V)[T_ctx - 1:]  # view that begins at row T_ctx-1 of sequence 0
        q = None
        if draft_logits is not None:
            q = draft_logits
            if isinstance(q, (list, tuple)):  # k arrays of (B, V), as `draft` returns them
                q = np.stack([np.asarray(_unwrap(x)) for x in q], axis=1)
        lens, toks = sampling.accept(self.ctx, start, q, draft.astype(np.int64), u_accept=u_accept,
                                     u_sample=u_sample, seed=seed, offset=offset, temperature=temperature,
                                     top_k=top_k, bonus=bonus, p_strides=(T * V, V), shape=(B, k, V))
        return toks.numpy(), lens.numpy(), None

    # -- training helper (out of the decode path; kept callable) --------------
    def draft_loss(self, draft_logits, target_tokens):
        """Mean cross-entropy over heads (speculative.py:316-348).  Host arithmetic: a training-side helper that
        is not part of the accelerated path.  Returns a scalar with `.data` and `.backward()`; `backward` fills
        `head.weight.grad` from the hidden rows of the last `draft` call."""
        target_tokens = np.asarray(_unwrap(target_tokens))
        if target_tokens.ndim != 2 or target_tokens.shape[1] != len(draft_logits):
            raise ValueError("target_tokens must be (B, k) with k equal to the number of draft heads")
        k = len(draft_logits)
        total, grads = 0.0, []
        for i, lg in enumerate(draft_logits):
            x = np.asarray(_unwrap(lg), dtype=np.float64)
            x = x - x.max(axis=-1, keepdims=True)
            e = np.exp(x)
            p = e / e.sum(axis=-1, keepdims=True)
            rows = np.arange(x.shape[0])
            total += float(np.mean(-np.log(p[rows, target_tokens[:, i]])))
            g = p.copy()
            g[rows, target_tokens[:, i]] -= 1.0
            grads.append(g / (x.shape[0] * k))
        return _Loss(total / k, self, grads)


class _Loss(float):
    """Scalar loss: a float with the `.data` / `.item()` / `.backward()` handles the reference's Tensor has."""

    def __new__(cls, value, decoder=None, grads=None):
        obj = super().__new__(cls, value)
        obj._decoder, obj._grads = decoder, grads
        return obj

    @property
    def data(self):
        return np.asarray(float(self), dtype=np.float32)

    def item(self):
        return float(self)

    def backward(self):
        dec = self._decoder
        h = getattr(dec, "_last_hidden", None)
        if h is None:
            raise RuntimeError("draft_loss.backward needs the hidden rows of a preceding draft() call")
        for head, g in zip(dec.draft_heads, self._grads):
            gw = (g.T @ np.asarray(h, dtype=np.float64)).astype(np.float32)     # (V, D)
            w = head.weight
            try:
                w.grad = gw if getattr(w, "grad", None) is None else w.grad + gw
            except AttributeError:
                pass


class no_grad:
    """Context manager with the name callers of the reference use around inference (verse_torch/tensor.py:99-133).
    This package records no autograd graph, so it changes nothing."""

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def _last_rows(ctx: Context, h: DeviceArray) -> DeviceArray:
    """(B, T, D) device array -> (B, D) copy of the last position."""
    B, T, D = h.shape
    if T == 1:
        return h.reshape(B, D)
    out = ctx.empty((B, D), np.float32)
    import ctypes as C
    for b in range(B):
        src = h.ptr + ((b * T + T - 1) * D) * 4
        ctx._check(ctx.lib.vn_d2d(ctx.handle, C.c_void_p(out.ptr + b * D * 4), C.c_void_p(src), D * 4))
    return out


def _split_heads(ctx: Context, logits: DeviceArray, B: int, k: int, V: int) -> List[DeviceArray]:
    """(B, k*V) -> k arrays (B, V)."""
    if B == 1:
        return [logits.reshape(k, V)[i:i + 1] for i in range(k)]
    import ctypes as C
    outs = []
    for i in range(k):                       # head i: B rows of V floats, k * V floats apart -> one pitched copy
        o = ctx.empty((B, V), np.float32)
        ctx._check(ctx.lib.vn_copy_2d(ctx.handle, C.c_void_p(o.ptr), V * 4, C.c_void_p(logits.ptr + i * V * 4), k * V * 4,
                                      V * 4, B))
        outs.append(o)
    return outs
