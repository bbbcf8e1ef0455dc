"""The C-ABI library: loads, exports every declared symbol, fails loudly without a GPU."""

import os
import re

import pytest

import versenext_b200 as vn
from versenext_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "vn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vn_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    lib = _lib.load()
    syms = declared_symbols()
    assert len(syms) >= 40
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/vn_b200.h but not exported"
        assert s in _lib.PROTOTYPES, f"{s} has no ctypes prototype"
    for s in _lib.PROTOTYPES:
        assert s in syms, f"{s} bound in Python but not declared in the header"


def test_version():
    assert _lib.load().vn_version() >= 100


def test_no_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(Exception) as e:
        vn.Context(0)
    assert "CUDA" in str(e.value) or "device" in str(e.value)
    with pytest.raises(Exception):
        vn.get_backend("cuda").matmul([[1.0]], [[1.0]])


def test_cpu_backend_is_not_offered():
    with pytest.raises(RuntimeError):
        vn.B200Backend("cpu")


def test_status_to_exception_mapping():
    assert _lib._EXC[_lib.VN_ERR_INVALID] is ValueError
    assert _lib._EXC[_lib.VN_ERR_OVERFLOW] is RuntimeError
    assert _lib._EXC[_lib.VN_ERR_INDEX] is IndexError


def test_speculative_decoder_constructor_contract():
    with pytest.raises(ValueError):
        vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=0)
    with pytest.raises(ValueError):
        vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=-1)
    d = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=3)
    assert len(d.draft_heads) == 3 and d.draft_heads[0].weight.data.shape == (16, 8)
    d.draft_heads[1].weight.data[5, :] = 10.0
    assert d.draft_heads[1].weight.data._dirty[0]
