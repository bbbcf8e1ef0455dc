"""Reader for the reference's `.vn` model container, streaming tensors to the device one at a time.

A `.vn` file is a ZIP archive (verse_torch/vn_format.py:1-60) holding `meta.json`, `config.yml` (YAML, or the JSON
subset of it) and the weights as `model.safetensors` or, where the writer had no safetensors, `model.npz`
(one `.npy` member per tensor, names with dots kept, :231-262).  `VNFileReader` here follows the reference's
reader (:527-660) in what it accepts -- format versions 1 and 2, both weight formats -- but never unpacks the
weights to a temporary file: the safetensors member is parsed in place (8-byte little-endian header length, a JSON
header with `dtype` / `shape` / `data_offsets` per tensor, then the raw bytes) and each tensor is handed out as soon
as it is read, so a multi-gigabyte checkpoint never sits on the host in full.
"""

from __future__ import annotations

import io
import json
import struct
import zipfile
from typing import Dict, Iterator, Optional, Tuple

import numpy as np

_ST_DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "I64": np.int64, "I32": np.int32,
              "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_, "U16": np.uint16, "U32": np.uint32,
              "U64": np.uint64}


def _bf16_to_f32(raw: bytes, shape) -> np.ndarray:
    u = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << np.uint32(16)
    return u.view(np.float32).reshape(shape)


class VNFileReader:
    def __init__(self, path: str):
        self.path = str(path)
        self._zf = zipfile.ZipFile(self.path, "r")
        self._names = set(self._zf.namelist())
        self._meta: Optional[dict] = None
        self.vn_format_version = 1

    # -- metadata -------------------------------------------------------------------------------------------
    def read_meta(self) -> dict:
        if self._meta is None:
            if "meta.json" not in self._names:
                raise ValueError(f"{self.path}: not a .vn file (no meta.json)")
            meta = json.loads(self._zf.read("meta.json").decode("utf-8"))
            version = meta.get("vn_format_version", 1)
            if version not in (1, 2):
                raise ValueError(f"unsupported .vn format version {version} (1 or 2 expected)")
            self.vn_format_version = version
            self._meta = meta
        return self._meta

    @property
    def weight_format(self) -> str:
        return self.read_meta().get("weight_format", "npz")

    def read_config(self) -> dict:
        if "config.yml" not in self._names:
            raise ValueError(f"{self.path}: no config.yml")
        text = self._zf.read("config.yml").decode("utf-8")
        try:
            import yaml
            loaded = yaml.safe_load(text)
        except ImportError:
            loaded = json.loads(text)
        return loaded if isinstance(loaded, dict) else {}

    # -- weights --------------------------------------------------------------------------------------------
    def iter_weights(self) -> Iterator[Tuple[str, np.ndarray]]:
        """(name, array) pairs in file order; float tensors of any stored width come out as float32, integer
        tensors (quantised weights) in their own dtype."""
        self.read_meta()
        if "model.safetensors" in self._names:
            yield from self._iter_safetensors()
        elif "model.npz" in self._names:
            yield from self._iter_npz()
        else:
            raise ValueError(f"{self.path}: no weights (model.safetensors / model.npz)")

    def read_weights(self) -> Dict[str, np.ndarray]:
        return dict(self.iter_weights())

    def _iter_safetensors(self):
        with self._zf.open("model.safetensors") as f:
            (hlen,) = struct.unpack("<Q", f.read(8))
            if hlen > (100 << 20):
                raise ValueError("implausible safetensors header length")
            header = json.loads(f.read(hlen).decode("utf-8"))
            entries = [(n, e) for n, e in header.items() if n != "__metadata__"]
            entries.sort(key=lambda ne: ne[1]["data_offsets"][0])
            pos = 0
            for name, e in entries:
                lo, hi = e["data_offsets"]
                if lo < pos:
                    raise ValueError(f"{name}: overlapping tensor data")
                if lo > pos:
                    f.read(lo - pos)
                raw = f.read(hi - lo)
                pos = hi
                if len(raw) != hi - lo:
                    raise ValueError(f"{name}: truncated tensor data")
                shape = tuple(e["shape"])
                if e["dtype"] == "BF16":
                    arr = _bf16_to_f32(raw, shape)
                else:
                    if e["dtype"] not in _ST_DTYPES:
                        raise ValueError(f"{name}: unsupported dtype {e['dtype']}")
                    arr = np.frombuffer(raw, dtype=_ST_DTYPES[e["dtype"]]).reshape(shape)
                    if arr.dtype in (np.float64, np.float16):
                        arr = arr.astype(np.float32)
                yield name, arr

    def _iter_npz(self):
        inner = zipfile.ZipFile(io.BytesIO(self._zf.read("model.npz")), "r")
        for entry in inner.namelist():
            if not entry.endswith(".npy"):
                continue
            with inner.open(entry) as f:
                arr = np.lib.format.read_array(f, allow_pickle=False)
            if arr.dtype in (np.float64, np.float16):
                arr = arr.astype(np.float32)
            yield entry[:-4], arr

    # -- optional members -----------------------------------------------------------------------------------
    def read_chat_template(self) -> Optional[str]:
        return self._zf.read("chat_template.jinja").decode("utf-8") if "chat_template.jinja" in self._names else None

    def read_tokenizer(self) -> Optional[dict]:
        return json.loads(self._zf.read("tokenizer.json").decode("utf-8")) if "tokenizer.json" in self._names else None

    def close(self):
        if self._zf is not None:
            self._zf.close()
            self._zf = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


_CTOR_KEYS = ("vocab_size", "dim", "n_layer", "n_head", "n_kv_head", "layer_pattern", "window_size",
              "num_global_tokens", "anchor_interval", "latent_dim", "use_alibi", "use_rope", "max_seq_len", "dropout",
              "rope_theta", "num_dense_parts", "num_experts_per_part", "top_k", "expert_hidden", "aux_loss_weight",
              "dense_part_names", "tie_weights", "mlp_hidden_multiple", "init_std", "residual_scale",
              "embedding_scale")


def load_vn(path: str, dtype: str = "f32", device: str = "cuda", **overrides):
    """A device-resident `VerseNexLM` from a `.vn` file (the reference's `CometSparkNexLM._load_vn`,
    verse_nex/cometspark.py:1122-1141): constructor arguments from `config.yml`, weights streamed tensor by tensor."""
    from .model import VerseNexLM
    with VNFileReader(path) as r:
        r.read_meta()
        cfg = {k: v for k, v in r.read_config().items() if k in _CTOR_KEYS}
        cfg.update(overrides)
        cfg.pop("init_std", None)
        model = VerseNexLM(dtype=dtype, device=device, **cfg)
        for name, arr in r.iter_weights():
            if name == "head.weight" and model.tie_weights:
                continue
            model.load_tensor(name, arr)
        model.finalize()
    return model
