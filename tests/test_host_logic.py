"""Host-side logic of the drop-in classes that needs no GPU (a recording stand-in replaces the device context)."""

import numpy as np
import pytest

import versenext_b200.speculative as S


class _FakeArray:
    def __init__(self, arr):
        self.arr = np.array(arr, copy=True)


class _FakeCtx:
    def __init__(self):
        self.uploads = 0

    def from_numpy(self, arr):
        self.uploads += 1
        return _FakeArray(arr)


def _decoder(V=16, D=8, k=4):
    dec = S.SpeculativeDecoder(dim=D, vocab_size=V, num_draft_heads=k, seed=0)
    dec._ctx = _FakeCtx()
    return dec


def test_head_weight_replaced_by_a_tensor_over_a_plain_ndarray():
    """The reference's own tests assign `head.weight = Tensor(ndarray)` (tests/test_speculative_decode.py:159-167)."""
    dec = _decoder()
    for i, head in enumerate(dec.draft_heads):
        w = np.zeros((16, 8), np.float32)          # a plain ndarray, not the tracked subclass
        w[10 + i, :] = 10.0
        head.weight = S.Tensor(w, requires_grad=True)
    dev = dec._weights()
    assert dev.arr.shape == (4 * 16, 8)
    for i in range(4):
        assert dev.arr[i * 16 + 10 + i, 0] == 10.0 and dev.arr[i * 16, 0] == 0.0
    # a plain ndarray cannot report in-place writes: it is uploaded again and the write is seen
    dec.draft_heads[0].weight.data[3, :] = 7.0
    assert dec._weights().arr[3, 0] == 7.0


def test_head_weight_zeros_like_of_the_tracked_array():
    dec = _decoder()
    for i, head in enumerate(dec.draft_heads):
        w = np.zeros_like(head.weight.data)        # what the reference test does: keeps the array subclass
        w[10 + i, :] = 10.0
        head.weight = S.Tensor(w)
    dev = dec._weights()
    for i in range(4):
        assert dev.arr[i * 16 + 10 + i, 0] == 10.0


def test_tracked_weights_upload_only_when_written():
    dec = _decoder()
    dec._weights()
    assert dec.ctx.uploads == 1
    dec._weights()
    assert dec.ctx.uploads == 1                    # nothing changed: the device copy is reused
    dec.draft_heads[1].weight.data[2, :] = 1.0     # __setitem__
    assert dec._weights().arr[16 + 2, 0] == 1.0 and dec.ctx.uploads == 2
    dec.draft_heads[2].weight.data *= 0.0          # in-place ufunc
    assert np.all(dec._weights().arr[32:48] == 0.0) and dec.ctx.uploads == 3
    np.add.at(dec.draft_heads[3].weight.data, (0, 0), 5.0)
    assert dec.ctx.uploads == 3 and dec._weights().arr[48, 0] != 0 and dec.ctx.uploads == 4
    dec.draft_heads[0].weight.data = np.ones((16, 8), np.float32)   # setter
    assert np.all(dec._weights().arr[:16] == 1.0) and dec.ctx.uploads == 5
    dec._weights()
    assert dec.ctx.uploads == 5


def test_head_weight_of_the_wrong_shape_is_rejected():
    import pytest
    dec = _decoder()
    dec.draft_heads[0].weight = S.Tensor(np.zeros((15, 8), np.float32))
    with pytest.raises(ValueError):
        dec._weights()


def test_delta_layer_pattern_and_synthetic_shapes(golden):
    """`build_verse_delta_pattern` of the package against the lists recorded from the reference, and the synthetic
    weight generator's tensor names and shapes for delta layers against the oracle's (= the reference's state_dict)."""
    import versenext_b200 as vn
    from versenext_b200 import synthetic
    from oracle import delta as OD
    from oracle import model as OM
    g = golden("delta_reference.npz")
    for n in (1, 5, 6, 9, 10, 14):
        assert vn.build_verse_delta_pattern(n) == list(g[f"pattern_{n}"])
    with pytest.raises(ValueError):
        vn.build_verse_delta_pattern(0)
    for tag in "abc":
        cfg, _ = OD.golden_case(tag)
        got = dict(synthetic._shapes(cfg.to_dict()))
        want = {n: tuple(s) for n, s in OM.param_shapes(cfg).items() if not (n == "head.weight" and cfg.tie_weights)}
        assert got == want
