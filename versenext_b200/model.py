"""`VerseNexLM` (= CometSparkNexLM) resident on the device.

Constructor keywords, attributes, `state_dict` names and the `forward` /
`__call__` / `generate` signatures follow verse_nex/cometspark.py:294-449,
:670-698 and :773-830.  `embedding_scale=True` adds the `tok_emb * sqrt(dim)`
of the CometSparkV05LM wrapper (spark/src/base_model.py:199-206).

Differences that the device path brings (all additive):
  * `dtype="f32" | "bf16"` selects the storage type of weights, GEMM inputs
    and the KV cache (accumulation, residual stream, softmax and logits stay
    float32);
  * layers of the delta attention kinds ("vda", "dsa", "kda", "gmla", verse_nex/delta_attention.py) compute the
    whole-sequence forward of those classes on the cache (masks from absolute positions; a GMLA module caches the
    K / V rebuilt from its latents);
  * `new_cache()` returns a `KVCache`; `forward_cached` runs T new positions
    (a chain, or a tree given `parents`) on top of it, which is what
    `SpeculativeDecoder.verify` re-computes from scratch in the reference
    (speculative.py:202-213).
Weights are not initialised here: load them with `load_state_dict` from a
reference `state_dict()` (name -> float32 ndarray, vnnn.py:235-285).
"""

from __future__ import annotations

import ctypes as C
import json
from typing import List, Optional

import numpy as np

from . import sampling
from .device import Context, DeviceArray, as_device

VALID_KINDS = ("trisparse", "mod", "vda", "dsa", "kda", "gmla")      # VerseNexBlock.VALID_KINDS, cometspark.py:110


def build_verse_delta_pattern(n_layer: int) -> List[str]:
    """Layer kinds of the delta architecture (verse_nex/delta_attention.py:1218-1247): fewer than 6 layers all
    "vda"; up to 9 four "vda" then "gmla"; from 10 on four "vda", "gmla" in between, two "dsa" at the end."""
    if n_layer < 1:
        raise ValueError(f"n_layer must be >= 1, got {n_layer}")
    if n_layer < 6:
        return ["vda"] * n_layer
    if n_layer < 10:
        return ["vda"] * 4 + ["gmla"] * (n_layer - 4)
    return ["vda"] * 4 + ["gmla"] * (n_layer - 6) + ["dsa"] * 2


def _ptr(a):
    return C.c_void_p(a.ptr) if a is not None else C.c_void_p(None)


def _as_quantised(v):
    """(packed, scale, qtype) when `v` is a linear in quantised form, else None."""
    if isinstance(v, tuple) and len(v) == 3 and isinstance(v[2], str):
        return v
    inner = getattr(v, "_qlin", v)          # QLinear module -> the QuantizedLinear it wraps
    if hasattr(inner, "packed") and hasattr(inner, "scale") and hasattr(inner, "qtype"):
        return inner.packed, inner.scale, inner.qtype
    return None


def _is_router_gate(name: str) -> bool:
    return name.endswith("router.gate.weight") or name.endswith("part_router.gate.weight")


def _dequantise_host(packed, scale, qtype):
    """q * scale as float32 (verse_torch/quantize.py:216-229, :260-275); used for the few small gate matrices only."""
    packed = np.asarray(packed)
    if qtype == "int8":
        q = packed.astype(np.float32)
    else:
        lo = (packed & 0x0F).astype(np.int16)
        hi = ((packed >> 4) & 0x0F).astype(np.int16)
        q = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.float32)
        q[..., 0::2] = np.where(lo >= 8, lo - 16, lo)
        q[..., 1::2] = np.where(hi >= 8, hi - 16, hi)
    sc = np.asarray(scale, dtype=np.float32).reshape(q.shape[0], -1)
    if sc.shape[1] > 1:
        return (q.reshape(q.shape[0], sc.shape[1], -1) * sc[..., None]).reshape(q.shape)
    return q * sc


class KVCache:
    """Per-layer K / V of shape (max_batch, max_seq, n_kv_head, head_dim) with per-sequence lengths.

    Same role and vocabulary as ParallelKVCache (verse_nex/kv_cache_parallel.py:42-283):
    `per_seq_lens`, `reset_seq`, `get`; overflow raises RuntimeError, a bad layer index IndexError.
    `commit` is new: it keeps a chosen subset of the entries appended by the last forward
    (accepted path) and drops the rest (rejected suffix) by compacting in place.
    """

    def __init__(self, model: "VerseNexLM", max_batch: int, max_seq: int, _view_of: Optional["KVCache"] = None,
                 _first: int = 0):
        self.model = model
        self.ctx = model.ctx
        self.max_batch, self.max_seq = int(max_batch), int(max_seq)
        self._parent = _view_of            # keeps the owning cache alive
        h = C.c_void_p()
        if _view_of is None:
            self.ctx._check(self.ctx.lib.vn_kv_create(model.handle, self.max_batch, self.max_seq, C.byref(h)))
        else:
            self.ctx._check(self.ctx.lib.vn_kv_view(_view_of.handle, int(_first), self.max_batch, C.byref(h)))
        self.handle = h

    def view(self, first: int, count: int = 1) -> "KVCache":
        """Sequences [first, first + count) of this cache as a cache of their own (shared memory): a serving loop
        prefills one free slot through it while the other sequences keep decoding."""
        if first < 0 or count < 1 or first + count > self.max_batch:
            raise IndexError(f"sequences [{first}, {first + count}) outside the cache's {self.max_batch}")
        return KVCache(self.model, count, self.max_seq, _view_of=self, _first=first)

    @property
    def per_seq_lens(self) -> np.ndarray:
        out = np.zeros(self.max_batch, dtype=np.int32)
        self.ctx._check(self.ctx.lib.vn_kv_lengths(self.handle, out.ctypes.data_as(C.c_void_p)))
        return out

    def set_lengths(self, lens):
        lens = np.ascontiguousarray(lens, dtype=np.int32)
        if lens.shape != (self.max_batch,):
            raise ValueError(f"lens must have shape ({self.max_batch},)")
        self.ctx._check(self.ctx.lib.vn_kv_set_lengths(self.handle, lens.ctypes.data_as(C.c_void_p)))

    def reset_seq(self, seq_idx: Optional[int] = None):
        self.ctx._check(self.ctx.lib.vn_kv_reset_seq(self.handle, -1 if seq_idx is None else int(seq_idx)))

    def reset(self):
        self.reset_seq(None)

    def commit(self, n_new: int, n_keep, keep_idx=None, keep_add: int = 0):
        """Keep `n_keep[b] + keep_add` of the `n_new` entries the last forward(s) appended to sequence b:
        the first ones (chain), or the slots listed in `keep_idx[b]` (tree path, ascending)."""
        nk = as_device(self.ctx, n_keep, np.int32)
        ki = as_device(self.ctx, keep_idx, np.int32) if keep_idx is not None else None
        stride = ki.shape[-1] if ki is not None else 0
        self.ctx._check(self.ctx.lib.vn_kv_commit(self.handle, int(n_new), _ptr(ki), stride, _ptr(nk), int(keep_add)))

    def get(self, layer_idx: int, seq_idx: int = 0, n_positions: Optional[int] = None):
        """(k, v) float32 ndarrays of shape (n_positions, n_kv_head, head_dim) for one sequence.  `layer_idx` counts
        K / V plane pairs: one per layer, three (dsa, kda, gmla) for a "vda" layer."""
        if n_positions is None:
            n_positions = int(self.per_seq_lens[seq_idx])
        m = self.model
        out = []
        for which in (0, 1):
            a = np.empty((n_positions, m.n_kv_head, m.head_dim), dtype=np.float32)
            self.ctx._check(self.ctx.lib.vn_kv_read(self.handle, int(layer_idx), int(seq_idx), which,
                                                    a.ctypes.data_as(C.c_void_p), int(n_positions)))
            out.append(a)
        return tuple(out)

    def __del__(self):
        try:
            if self.handle:
                self.ctx.lib.vn_kv_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


class VerseNexLM:
    def __init__(self, vocab_size: int, dim: int, n_layer: int, n_head: int, n_kv_head: Optional[int] = None,
                 layer_pattern: Optional[List[str]] = None, window_size: int = 512, num_global_tokens: int = 64,
                 anchor_interval: int = 128, latent_dim=None, use_alibi: bool = True, use_rope: bool = False,
                 max_seq_len: int = 2048, dropout: float = 0.0, rope_theta: float = 10000.0,
                 num_dense_parts: int = 5, num_experts_per_part: int = 8, top_k: int = 3,
                 expert_hidden: Optional[int] = None, aux_loss_weight: float = 0.01, dense_part_names=None,
                 tie_weights: bool = True, mlp_hidden_multiple: int = 4, init_std: float = 0.02,
                 residual_scale=None, embedding_scale: bool = False, dtype: str = "f32", device: str = "cuda"):
        if layer_pattern is None:
            layer_pattern = ["trisparse"] * n_layer
        if len(layer_pattern) != n_layer:
            raise ValueError(f"layer_pattern length ({len(layer_pattern)}) must equal n_layer ({n_layer})")
        for i, k in enumerate(layer_pattern):
            if k not in VALID_KINDS:
                raise ValueError(f"layer_pattern[{i}]={k!r} is not available on this backend {VALID_KINDS}")
        if dtype not in ("f32", "bf16"):
            raise ValueError("dtype must be 'f32' or 'bf16'")
        self.vocab_size, self.dim, self.n_layer, self.n_head = int(vocab_size), int(dim), int(n_layer), int(n_head)
        self.n_kv_head = int(n_kv_head) if n_kv_head is not None else int(n_head)
        self.head_dim = self.dim // self.n_head
        self.layer_pattern = list(layer_pattern)
        self.tie_weights = bool(tie_weights)
        self.max_seq_len = int(max_seq_len)
        self.window_size = int(window_size)
        self.anchor_interval = int(anchor_interval)
        self.latent_dim = None if latent_dim is None else int(latent_dim)
        if self.anchor_interval < 1:
            raise ValueError(f"anchor_interval must be >= 1, got {anchor_interval}")
        self.use_rope, self.use_alibi = bool(use_rope), bool(use_alibi)
        self.rope_theta = float(rope_theta)
        self.embedding_scale = bool(embedding_scale)
        self.dtype = dtype
        self.aux_loss_weight = aux_loss_weight
        self._config = dict(vocab_size=self.vocab_size, dim=self.dim, n_layer=self.n_layer, n_head=self.n_head,
                            n_kv_head=self.n_kv_head, layer_pattern=self.layer_pattern, window_size=int(window_size),
                            num_global_tokens=int(num_global_tokens), anchor_interval=self.anchor_interval,
                            latent_dim=self.latent_dim, use_alibi=self.use_alibi, use_rope=self.use_rope,
                            max_seq_len=self.max_seq_len, rope_theta=self.rope_theta,
                            num_dense_parts=int(num_dense_parts), num_experts_per_part=int(num_experts_per_part),
                            top_k=int(top_k), expert_hidden=expert_hidden, tie_weights=self.tie_weights,
                            mlp_hidden_multiple=int(mlp_hidden_multiple), embedding_scale=self.embedding_scale,
                            dtype=dtype)
        from .backend import _parse_index
        self.ctx = Context.get(_parse_index(device))
        h = C.c_void_p()
        self.ctx._check(self.ctx.lib.vn_model_create(self.ctx.handle, json.dumps(self._config).encode(), C.byref(h)))
        self.handle = h
        self._finalized = False
        self._scratch_cache: Optional[KVCache] = None

    @classmethod
    def from_pretrained(cls, path: str, dtype: str = "f32", device: str = "cuda", **overrides) -> "VerseNexLM":
        """A model from a `.vn` file, or from a directory holding `model.vn` (CometSparkNexLM.from_pretrained,
        verse_nex/cometspark.py:1077-1141).  The reference's pickle formats (`.pt`) are not read."""
        import os
        from .vn_file import load_vn
        p = str(path)
        if os.path.isdir(p):
            p = os.path.join(p, "model.vn")
            if not os.path.exists(p):
                raise FileNotFoundError(f"no model.vn in {path}")
        elif not p.endswith(".vn"):
            raise ValueError("only the .vn container is read (pickled .pt checkpoints are not)")
        return load_vn(p, dtype=dtype, device=device, **overrides)

    # -- reference-compatible helpers -----------------------------------------
    def get_config(self) -> dict:
        return dict(self._config)

    def eval(self):
        return self

    def param_bytes(self) -> int:
        n = C.c_uint64()
        self.ctx._check(self.ctx.lib.vn_model_param_bytes(self.handle, C.byref(n)))
        return int(n.value)

    def head_columns(self, hidden, v_lo: int, n_cols: int) -> DeviceArray:
        """Logits of vocabulary columns [v_lo, v_lo + n_cols) for final-norm hidden rows (R, dim): the LM head of a
        rank that owns only those columns."""
        h = as_device(self.ctx, hidden, np.float32)
        R = h.size // self.dim
        out = self.ctx.empty((R, n_cols), np.float32)
        self.ctx._check(self.ctx.lib.vn_model_head(self.handle, _ptr(h), R, int(v_lo), int(n_cols), _ptr(out), n_cols))
        return out

    def check(self):
        """Raise what the forwards since the last check ran into on the device: IndexError for a token id outside
        the vocabulary (as NumPy indexing does in the reference, vnnn.py:453-460), RuntimeError for a kernel
        wait that ran out.  Synchronises the stream."""
        self.ctx._check(self.ctx.lib.vn_model_status(self.handle, None, None))

    def load_tensor(self, name: str, array):
        a = np.ascontiguousarray(np.asarray(array), dtype=np.float32)
        shape = (C.c_int64 * max(a.ndim, 1))(*(a.shape if a.ndim else (1,)))
        self.ctx._check(self.ctx.lib.vn_model_load_tensor(self.handle, name.encode(), a.ctypes.data_as(C.c_void_p),
                                                          max(a.ndim, 1), shape))
        self._finalized = False

    def load_state_dict(self, sd: dict, strict: bool = True):
        """name -> float32 array (vnnn.py:235-285).  A value may also be an already quantised linear: an object
        with `packed`, `scale` and `qtype` (the reference's QuantizedLinear, quantize.py:382-440, or the QLinear
        module that wraps one in `_qlin`, compress.py:739-756) or a `(packed, scale, qtype)` tuple; those go to
        the device as they are (`load_quant_tensor`)."""
        quantised = {n: v for n, v in sd.items() if _as_quantised(v) is not None}
        for name, value in sd.items():
            if name in quantised:
                continue
            if name == "head.weight" and self.tie_weights and not quantised:
                continue
            self.load_tensor(name, getattr(value, "data", value))
        for name, value in quantised.items():
            packed, scale, qtype = _as_quantised(value)
            if _is_router_gate(name):
                # router gates stay float32 on the device: a quantised gate is expanded here (q * scale)
                self.load_tensor(name, _dequantise_host(packed, scale, qtype))
            else:
                self.load_quant_tensor(name, packed, scale, qtype)
        self.finalize()

    def load_quant_tensor(self, name: str, packed, scale, qtype: str = "int4"):
        """One linear in its quantised form, exactly the bytes and scales given (no re-quantisation).
        packed: int8 (out, in) for "int8", uint8 (out, in/2) for "int4" / "int4g128"; scale: (out, 1) or (out,)
        float32, (out, in/128) for "int4g128"."""
        packed = np.ascontiguousarray(packed)
        rows = packed.shape[0]
        K = packed.shape[1] if qtype == "int8" else packed.shape[1] * 2
        if qtype == "int8" and packed.dtype != np.int8 or qtype != "int8" and packed.dtype != np.uint8:
            raise ValueError(f"{name}: packed has dtype {packed.dtype}, expected int8 (int8) or uint8 (int4 schemes)")
        sc = np.ascontiguousarray(np.asarray(scale, dtype=np.float32).reshape(rows, -1))
        want = (K + 127) // 128 if qtype == "int4g128" else 1
        if sc.shape[1] != want:
            raise ValueError(f"{name}: scale has {sc.shape[1]} values per row, expected {want}")
        self.ctx._check(self.ctx.lib.vn_model_load_quant_tensor(
            self.handle, name.encode(), qtype.encode(), packed.ctypes.data_as(C.c_void_p),
            sc.ctypes.data_as(C.c_void_p), rows, K))
        self.quantized = qtype
        self._finalized = False

    def read_quant(self, name: str):
        """(q, scale) of one linear of a quantised model as they sit on the device: int8 (out, in) or packed uint8
        (out, in/2), scale float32 (out, 1) or (out, in/128)."""
        qtype = getattr(self, "quantized", None)
        if qtype is None:
            raise ValueError("the model holds no quantised weights")
        rows, K = self.linear_shape(name)
        q = np.empty((rows, K) if qtype == "int8" else (rows, K // 2), np.int8 if qtype == "int8" else np.uint8)
        sc = np.empty((rows, (K + 127) // 128 if qtype == "int4g128" else 1), np.float32)
        self.ctx._check(self.ctx.lib.vn_model_read_quant(self.handle, name.encode(), q.ctypes.data_as(C.c_void_p),
                                                         q.nbytes, sc.ctypes.data_as(C.c_void_p), sc.size))
        return q, sc

    def linear_shape(self, name: str):
        """(out_features, in_features) of a linear given by its state_dict name."""
        D, hd = self.dim, self.head_dim
        qd, kvd = self.n_head * hd, self.n_kv_head * hd
        c = self._config
        hidden = ((c["mlp_hidden_multiple"] * D * 2.0 / 3.0 + 63) // 64) * 64
        eh = c["expert_hidden"] or max(int(D * 8.0 / 3.0 / 64.0) * 64, 64)
        leaf = name.split(".")[-2]
        if name == "head.weight":
            return self.vocab_size, D
        if ".experts." in name:
            return {"w_gate": (eh, D), "w_up": (eh, D), "w_down": (D, eh)}[leaf]
        lat = self.latent_dim or kvd
        table = {"wq": (qd, D), "wk": (kvd, D), "wv": (kvd, D), "proj": (D, qd), "w_gate": (int(hidden), D),
                 "w_up": (int(hidden), D), "w_down": (D, int(hidden)),
                 "w_kv_down": (lat, D), "w_k_up": (kvd, lat), "w_v_up": (kvd, lat)}      # GMLA (delta_attention.py:861-863)
        if leaf not in table:
            raise ValueError(f"{name} is not a linear of this model")
        return table[leaf]

    def finalize(self):
        if self.use_rope:
            # RoPE table with the reference's own NumPy expression (tri_sparse_attn.py:169-180)
            half = self.head_dim // 2
            rows = max(self.max_seq_len, 16) * 2
            i = np.arange(half, dtype=np.float32)
            inv_freq = 1.0 / (self.rope_theta ** (2.0 * i / self.head_dim))
            ang = np.outer(np.arange(rows, dtype=np.float32), inv_freq)
            self.load_tensor("rope.cos", np.cos(ang).astype(np.float32))
            self.load_tensor("rope.sin", np.sin(ang).astype(np.float32))
        self.ctx._check(self.ctx.lib.vn_model_finalize(self.handle))
        self._finalized = True

    def quantize(self, scheme: str = "int8"):
        """Weight-only quantisation of every Linear of the blocks and of the LM head, on the device.

        "int8" and "int4" are the reference's per-output-channel schemes (verse_torch/quantize.py:187-258:
        scale = max|w| / 127 or / 7, round-half-even, INT4 packed two per byte with the even index in the low
        nibble); "int4g128" keeps one bf16 scale per 128 input features.  The LM head gets its own quantised
        copy (as compress.py:817-822 un-ties it); the embedding table and the router gates stay dense.
        bf16 models only.  The dense weights are released: the model cannot be reloaded afterwards."""
        if not self._finalized:
            self.finalize()
        self.ctx._check(self.ctx.lib.vn_model_quantize(self.handle, scheme.encode()))
        self.quantized = scheme
        return self

    def new_cache(self, max_batch: int, max_seq: Optional[int] = None) -> KVCache:
        return KVCache(self, max_batch, max_seq if max_seq is not None else self.max_seq_len)

    # -- forward -----------------------------------------------------------------
    def forward_cached(self, tokens, cache: KVCache, parents=None, last_only: bool = False,
                       want_logits: bool = True, want_hidden: bool = False, slot_offset: int = 0,
                       out_logits: Optional[DeviceArray] = None, out_hidden: Optional[DeviceArray] = None):
        """T new positions per sequence on top of `cache` (appended, not yet committed).

        tokens (B, T) int64 host or device; parents: list of T tree parents (-1 = child of the last
        committed token) or None for a chain.  Returns logits (B, T | 1, V) and / or hidden."""
        if not self._finalized:
            self.finalize()
        tok = as_device(self.ctx, tokens, np.int64)
        B, T = tok.shape
        rows = 1 if last_only else T
        logits = hidden = None
        if want_logits:
            logits = out_logits if out_logits is not None else self.ctx.empty((B, rows, self.vocab_size), np.float32)
        if want_hidden:
            hidden = out_hidden if out_hidden is not None else self.ctx.empty((B, rows, self.dim), np.float32)
        par = None
        if parents is not None:
            par = np.ascontiguousarray(parents, dtype=np.int32)
            if par.shape != (T,):
                raise ValueError("parents must list one parent per new position")
        self.ctx._check(self.ctx.lib.vn_model_forward(
            self.handle, cache.handle, _ptr(tok), B, T,
            par.ctypes.data_as(C.c_void_p) if par is not None else None, _ptr(hidden), _ptr(logits),
            int(bool(last_only)), int(slot_offset)))
        if want_logits and want_hidden:
            return logits, hidden
        return logits if want_logits else hidden

    def forward(self, idx):
        """Whole-sequence forward from position 0, logits (B, T, V) -- CometSparkNexLM.forward."""
        from .speculative import Tensor, _unwrap
        ids = _unwrap(idx)
        ids = ids if isinstance(ids, DeviceArray) else np.asarray(ids, dtype=np.int64)
        if ids.ndim == 1:
            ids = ids.reshape(1, -1)
        B, T = ids.shape
        c = self._scratch_cache
        if c is None or c.max_batch < B or c.max_seq < T:
            self._scratch_cache = c = self.new_cache(max(B, 1), max(T, self.max_seq_len))
        c.reset()
        out = Tensor(self.forward_cached(ids, c))
        self.check()
        return out

    __call__ = forward

    def forward_recurrent(self, input_ids, states=None):
        """One decoding step, CometSparkNexLM.forward_recurrent (cometspark.py:737-767): input_ids (B, 1) ->
        (logits (B, 1, V), new_states) with one state entry per layer.

        The reference threads per-layer dicts of grown K/V arrays through the call; here every entry of the
        returned list is the same device-resident `KVCache`, extended in place by the step (a list taken from an
        earlier step therefore sees the later tokens too).  `states=None` starts a fresh cache of `max_seq_len`
        positions; more than one token per call raises AssertionError as the reference's attention does
        (tri_sparse_attn.py:635), a full cache raises RuntimeError."""
        from .speculative import Tensor, _unwrap
        ids = _unwrap(input_ids)
        ids = ids if isinstance(ids, DeviceArray) else np.asarray(ids, dtype=np.int64)
        if ids.ndim == 1:
            ids = ids.reshape(-1, 1)
        B, T = ids.shape
        assert T == 1, f"forward_recurrent takes one token per sequence, got T={T}"
        if states is None:
            cache = self.new_cache(B, self.max_seq_len)
        else:
            cache = states[0]
            if not isinstance(cache, KVCache) or cache.max_batch < B:
                raise ValueError("states must be the list returned by an earlier forward_recurrent call of this batch")
        if int(cache.per_seq_lens[:B].max()) + 1 > cache.max_seq:
            raise RuntimeError(f"KV cache overflow: {cache.max_seq} positions are in use")
        self._set_recurrent(True)        # the ALiBi path of the one-token step sees the last window_size keys only
        try:
            logits = self.forward_cached(ids, cache)
        finally:
            self._set_recurrent(False)
        cache.commit(1, np.ones(B, np.int32))
        self.check()
        return Tensor(logits), [cache] * self.n_layer

    def _set_recurrent(self, on: bool):
        self.ctx._check(self.ctx.lib.vn_model_set_recurrent(self.handle, int(bool(on))))

    def set_fused_stack(self, on: bool):
        """Run the whole layer stack as one cooperative kernel where the model allows it (small all-TriSparse bf16
        models: the draft).  Off by default: the chain of separate kernels is as fast on B200."""
        self.ctx._check(self.ctx.lib.vn_model_set_fused_stack(self.handle, int(bool(on))))

    # -- generate (cometspark.py:773-830) -------------------------------------------
    def generate(self, idx, max_new_tokens: Optional[int] = None, temperature: float = 1.0,
                 top_k: Optional[int] = None, eos_id: Optional[int] = None, max_safe_limit: int = 100_000,
                 seed: int = 0, draft: Optional["VerseNexLM"] = None, k: int = 4) -> np.ndarray:
        """Autoregressive generation with the KV cache.  As in the reference, `temperature == 1.0 and
        top_k is None` means GREEDY decoding on the recurrent route (cometspark.py:817-818, :832-866), with that
        route's two peculiarities kept: the last prompt token is fed twice, and the ALiBi path sees the last
        `window_size` keys.  Any other setting follows `_generate_with_logits` (:868-915): whole-sequence
        semantics, arg-max for `temperature <= 0`, else a draw from softmax(logits / T) over the top-k with
        uniforms from Philox(seed)."""
        from .speculative import _unwrap
        ids = np.asarray(_unwrap(idx))
        if ids.ndim == 1:
            ids = ids[None, :]
        ids = ids.astype(np.int64)
        limit = max_safe_limit if max_new_tokens is None else int(max_new_tokens)
        recurrent = temperature == 1.0 and top_k is None     # the reference's greedy + recurrent route (:817-818)
        if draft is not None:
            return self._generate_speculative(ids, limit, temperature, top_k, eos_id, seed, draft, k, recurrent)
        B, T0 = ids.shape
        cap = T0 + min(limit, 1 << 20) + 2
        if self.use_rope:
            cap = min(cap, 2 * max(self.max_seq_len, 16))   # rows of the RoPE table
        cache = self.new_cache(B, cap)
        out = [ids]
        self._set_recurrent(recurrent)
        try:
            logits = self.forward_cached(ids, cache, last_only=True)
            cache.commit(T0, np.full(B, T0, np.int32))
            if recurrent and limit > 0:
                # the reference warms its state up with the whole prompt and then feeds the LAST PROMPT TOKEN ONCE
                # MORE; the logits of that second pass pick the first new token (cometspark.py:848-856)
                logits = self.forward_cached(ids[:, -1:], cache, last_only=True)
                cache.commit(1, np.ones(B, np.int32))
            for step in range(limit):
                lg = logits.reshape(B, self.vocab_size)
                if recurrent or temperature <= 0:
                    nxt = sampling.argmax(self.ctx, lg)
                else:
                    nxt = sampling.sample(self.ctx, lg, temperature=temperature, top_k=top_k or 0, seed=seed,
                                          offset=step)
                host = nxt.numpy()
                out.append(host[:, None])
                if eos_id is not None and np.all(host == eos_id):
                    break
                if step + 1 == limit:
                    break
                logits = self.forward_cached(nxt.reshape(B, 1), cache, last_only=True)
                cache.commit(1, np.ones(B, np.int32))
        finally:
            self._set_recurrent(False)
        self.check()
        res = np.concatenate(out, axis=1)
        if eos_id is not None and res.shape[1] > 0 and not np.all(res[:, -1] == eos_id):
            res = np.concatenate([res, np.full((B, 1), eos_id, dtype=res.dtype)], axis=1)
        return res

    def _generate_speculative(self, ids, limit, temperature, top_k, eos_id, seed, draft, k, recurrent):
        """`generate` through the speculative engine (`draft` proposes k tokens per round, this model verifies them).
        Greedy settings give exactly the tokens of the plain loop above, in fewer target forwards; sampling settings
        draw from the same distribution (rejection sampling) but not the same Philox stream."""
        from .engine import SpecEngine
        B, T0 = ids.shape
        greedy = recurrent or temperature <= 0
        prompts = ids
        if recurrent:
            # the recurrent route feeds the last prompt token twice (cometspark.py:848-856): it simply is part of the
            # context the first new token is predicted from
            prompts = np.concatenate([ids, ids[:, -1:]], axis=1)
        if prompts.shape[1] < 2:
            prompts = np.concatenate([prompts[:, :1], prompts], axis=1) if not recurrent else prompts
        if prompts.shape[1] < 2:
            raise ValueError("speculative generation needs at least two context tokens")
        T1 = prompts.shape[1]
        limit = min(limit, 1 << 20)
        eng = SpecEngine(self, draft, max_batch=B, max_seq=T1 + limit + 2 * (k + 1) + 2, k=k,
                         temperature=0.0 if greedy else temperature, top_k=0 if greedy else (top_k or 0), seed=seed,
                         bonus=True, max_new_tokens=limit)
        self._set_recurrent(recurrent)
        draft._set_recurrent(recurrent)
        try:
            out, _ = eng.generate(prompts, limit, eos_id=eos_id)
        finally:
            self._set_recurrent(False)
            draft._set_recurrent(False)
        res = np.concatenate([ids, out[:, T1:]], axis=1)
        if eos_id is not None:
            new = res[:, T0:]
            stop = np.flatnonzero(np.all(new == eos_id, axis=0))     # the plain loop stops when every row emits EOS
            if stop.size:
                res = res[:, :T0 + int(stop[0]) + 1]
            if res.shape[1] > 0 and not np.all(res[:, -1] == eos_id):
                res = np.concatenate([res, np.full((B, 1), eos_id, dtype=res.dtype)], axis=1)
        return res

    def __del__(self):
        try:
            self._scratch_cache = None
            if self.handle:
                self.ctx.lib.vn_model_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


CometSparkNexLM = VerseNexLM
