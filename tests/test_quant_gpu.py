"""Integer parity of the weight-only quantisation path (bit-exact: bytes and scales).

  * the device quantiser against the arrays the REAL reference functions returned
    (tests/golden/quant_reference.npz: quantize_int8 / quantize_int4 of verse_torch/quantize.py:187-258);
  * the quantised tensors a device model holds after `quantize()`, read back through the C ABI, against the
    oracle's quantiser on the same bf16 weights;
  * ingestion: linears given as (packed, scale) -- the form a reference QuantizedLinear keeps them in -- land on
    the device unchanged and drive the same forward as quantising on the device.
"""

import numpy as np
import pytest

from oracle import model as OM
from oracle import quant as OQ

pytestmark = pytest.mark.gpu


def _ctx():
    import versenext_b200 as vn
    return vn.Context.get(0)


def test_device_quantiser_equals_reference_bytes(golden):
    import versenext_b200 as vn
    g = golden("quant_reference.npz")
    ctx = _ctx()
    q8, s8 = vn.quant.quantize(ctx, g["w"], "int8")
    assert q8.dtype == np.int8 and q8.shape == g["q8"].shape and s8.shape == g["s8"].shape
    np.testing.assert_array_equal(q8.numpy(), g["q8"])
    np.testing.assert_array_equal(s8.numpy().view(np.uint32), g["s8"].view(np.uint32))
    p4, s4 = vn.quant.quantize(ctx, g["w"], "int4")
    assert p4.dtype == np.uint8 and p4.shape == g["p4"].shape
    np.testing.assert_array_equal(p4.numpy(), g["p4"])
    np.testing.assert_array_equal(s4.numpy().view(np.uint32), g["s4"].view(np.uint32))


@pytest.mark.parametrize("rows,K", [(1, 64), (37, 192), (130, 2752), (5, 7), (3, 129)])
def test_device_quantiser_equals_oracle_on_ragged_shapes(rows, K):
    """Odd in_features (INT4 pads the last high nibble with zero), all-zero rows (scale 1/qmax), rows whose
    maximum is negative, values that land exactly between two steps (round half to even)."""
    import versenext_b200 as vn
    rng = np.random.default_rng(rows * 1000 + K)
    w = rng.normal(0, 0.05, (rows, K)).astype(np.float32)
    w[0] = 0.0
    if rows > 1:
        w[1] = -np.abs(w[1])
        w[1, 0] = -1.0                           # max |w| = 1: scale = 1/127 or 1/7
        if K >= 4:
            w[1, 1:4] = np.array([2.5 / 7.0, -3.5 / 127.0, 0.5 / 127.0], np.float32)   # halves: ties to even
    ctx = _ctx()
    for scheme in ("int8", "int4"):
        q, s = vn.quant.quantize(ctx, w, scheme)
        wq, ws = (OQ.quantize_int8 if scheme == "int8" else OQ.quantize_int4)(w)
        np.testing.assert_array_equal(q.numpy(), wq)
        np.testing.assert_array_equal(s.numpy().view(np.uint32), ws.view(np.uint32))
    if K % 2 == 0:
        q, s = vn.quant.quantize(ctx, w, "int4g128")
        wq, ws = OQ.quantize_int4_g128(w)
        np.testing.assert_array_equal(q.numpy(), wq)
        np.testing.assert_array_equal(s.numpy().view(np.uint32), np.ascontiguousarray(ws).view(np.uint32))


def _mini():
    cfg = OM.mate_config(vocab_size=320, dim=128, n_layer=2, n_head=4, n_kv_head=2, window_size=16,
                         num_global_tokens=8, max_seq_len=128, init_std=0.08, num_dense_parts=2,
                         num_experts_per_part=2, top_k=1, expert_hidden=192, mlp_hidden_multiple=3)
    sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=31, gate_std=1.0).items()}
    return cfg, sd


def _build(cfg, sd=None):
    import versenext_b200 as vn
    kw = cfg.to_dict()
    kw.pop("init_std")
    m = vn.VerseNexLM(dtype="bf16", **kw)
    if sd is not None:
        m.load_state_dict(sd)
    return m


def _linear_names(sd):
    return [n for n, w in sd.items() if w.ndim == 2 and n.endswith(".weight") and "global_tokens" not in n
            and "router" not in n and n != "tok_emb.weight"]


def _oracle_quant(w, scheme):
    if scheme == "int8":
        return OQ.quantize_int8(w)
    if scheme == "int4":
        return OQ.quantize_int4(w)
    p, s = OQ.quantize_int4_g128(w)
    return p, np.ascontiguousarray(s)


@pytest.mark.parametrize("scheme", ["int8", "int4", "int4g128"])
def test_model_quantised_tensors_read_back_bit_exact(scheme):
    """Every linear of a model quantised on the device -- incl. the stacked q|k|v, the interleaved gate|up, the
    per-expert matrices and the head's own copy -- holds the oracle's bytes and scales."""
    cfg, sd = _mini()
    m = _build(cfg, sd)
    m.quantize(scheme)
    names = _linear_names(sd) + ["head.weight"]
    for n in names:
        w = sd["tok_emb.weight"] if n == "head.weight" else sd[n]
        q, s = m.read_quant(n)
        wq, ws = _oracle_quant(w, scheme)
        np.testing.assert_array_equal(q, wq, err_msg=n)
        np.testing.assert_array_equal(s.view(np.uint32), ws.reshape(s.shape).view(np.uint32), err_msg=n)
    with pytest.raises(ValueError):
        m.read_quant("blocks.0.norm1.weight")


class _QuantLinear:
    """The attributes a reference QuantizedLinear exposes (verse_torch/quantize.py:382-440)."""

    def __init__(self, w, qtype):
        self.qtype = qtype
        self.packed, self.scale = (OQ.quantize_int8 if qtype == "int8" else OQ.quantize_int4)(w)
        self.w_shape = w.shape


@pytest.mark.parametrize("scheme", ["int8", "int4"])
def test_prequantised_linears_load_without_requantising(scheme):
    """A compressed reference model keeps every Linear as packed bytes + per-row scales (router gates included).
    Loading those gives (a) the very bytes back, (b) the forward of a model quantised on the device, bit for bit."""
    cfg, sd = _mini()
    ref = _build(cfg, sd)
    ref.quantize(scheme)
    toks = np.random.default_rng(8).integers(0, 320, (2, 30))
    cache = ref.new_cache(2, 64)
    want = ref.forward_cached(toks, cache).numpy()

    compressed = {}
    for n, w in sd.items():
        compressed[n] = _QuantLinear(w, scheme) if n in _linear_names(sd) else w
    compressed["head.weight"] = _QuantLinear(sd["tok_emb.weight"], scheme)
    # a value that is NOT what quantising would give: proves the bytes are taken as they are
    odd = compressed["blocks.1.attn.proj.weight"]
    odd.packed = odd.packed.copy()
    odd.packed[3, 5] ^= 0x11
    m = _build(cfg)
    m.load_state_dict(compressed)
    q, s = m.read_quant("blocks.1.attn.proj.weight")
    np.testing.assert_array_equal(q, odd.packed)
    np.testing.assert_array_equal(s, odd.scale)
    for n in ("blocks.0.attn.wk.weight", "blocks.1.ffn.w_up.weight", "head.weight"):
        q, s = m.read_quant(n)
        np.testing.assert_array_equal(q, compressed[n].packed, err_msg=n)
        np.testing.assert_array_equal(s, compressed[n].scale, err_msg=n)
    # same forward as the device-quantised model once the flipped byte is put back
    m2 = _build(cfg)
    odd.packed[3, 5] ^= 0x11
    m2.load_state_dict(compressed)
    got = m2.forward_cached(toks, m2.new_cache(2, 64)).numpy()
    np.testing.assert_array_equal(got, want)
    with pytest.raises(ValueError):
        m2.load_tensor("blocks.0.attn.wq.weight", sd["blocks.0.attn.wq.weight"])


def test_quantised_router_gate_is_expanded_on_the_host_and_mixed_loading_is_rejected():
    cfg, sd = _mini()
    gate = [n for n in sd if n.endswith("part_router.gate.weight")][0]
    mixed = dict(sd)
    q, s = OQ.quantize_int8(sd[gate])
    mixed[gate] = (q, s, "int8")
    for n in _linear_names(sd):
        mixed[n] = _QuantLinear(sd[n], "int8")
    mixed["head.weight"] = _QuantLinear(sd["tok_emb.weight"], "int8")
    m = _build(cfg)
    m.load_state_dict(mixed)              # gate dequantised on the host, every linear taken as bytes
    assert m.quantized == "int8"
    # dense linears first, then a quantised one: refused
    m3 = _build(cfg)
    m3.load_tensor("blocks.0.attn.wq.weight", sd["blocks.0.attn.wq.weight"])
    with pytest.raises(ValueError):
        m3.load_quant_tensor("blocks.0.attn.wk.weight", *OQ.quantize_int8(sd["blocks.0.attn.wk.weight"]), "int8")
