"""The scenarios of the reference's own test files for this path, run against the drop-in.

Each test restates one case of the reference's tests/test_speculative_decode.py (12 cases, cited per test) or of
the operator block of tests/test_device_backend.py:56-207, with `versenext_b200` imported where the reference
imports `verse_torch` / `verse_nex` -- the substitution a maintainer makes when switching.  Constants (dims,
vocabulary, forced tokens, contexts) are the reference's; the expected outcomes are the ones its assertions pin.
"""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vn():
    import versenext_b200
    return versenext_b200


class ControlledMainModel:
    """Embedding + linear head whose per-position logits can be overridden (the reference's FakeMainModel,
    tests/test_speculative_decode.py:36-73): returns (logits, hidden)."""

    def __init__(self, vn, vocab_size=16, dim=8, next_token_logits=None):
        rng = np.random.RandomState(0)
        self.vn, self.V, self.D = vn, vocab_size, dim
        self.E = rng.randn(vocab_size, dim).astype(np.float32)
        self.W = rng.randn(dim, vocab_size).astype(np.float32)
        self.table = next_token_logits

    def __call__(self, idx):
        ids = np.asarray(idx.data).astype(np.int64)
        hidden = self.E[ids]
        if self.table is not None:
            T = ids.shape[1]
            logits = np.broadcast_to(self.table[None, :T, :], (ids.shape[0], T, self.V)).astype(np.float32).copy()
        else:
            logits = hidden @ self.W
        return self.vn.Tensor(logits, requires_grad=False), self.vn.Tensor(hidden, requires_grad=False)


def _table(targets, T_ctx=3, V=16):
    t = np.full((32, V), -10.0, dtype=np.float32)
    for i, tok in enumerate(targets):
        t[T_ctx - 1 + i, tok] = 10.0
    return t


def _force_heads(vn, dec, tokens):
    """Exactly the reference tests' way of steering a head: a fresh array assigned as `head.weight = Tensor(...)`."""
    for head, tok in zip(dec.draft_heads, tokens):
        w = np.zeros_like(head.weight.data)
        w[tok, :] = 10.0
        head.weight = vn.Tensor(w, requires_grad=True)


# ---- tests/test_speculative_decode.py:81-132 ------------------------------------------------------------------
def test_draft_k4_candidate_shape(vn):
    dec = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=4)
    hidden = vn.Tensor(np.random.randn(1, 1, 8).astype(np.float32), requires_grad=False)
    tokens, logits = dec.draft(hidden)
    assert tokens.shape == (1, 4) and len(logits) == 4
    for lg in logits:
        assert lg.data.shape == (1, 16)
    assert np.all(tokens >= 0) and np.all(tokens < 16)


def test_draft_various_hidden_shapes(vn):
    dec = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=4)
    assert dec.draft(vn.Tensor(np.random.randn(2, 8).astype(np.float32)))[0].shape == (2, 4)
    assert dec.draft(vn.Tensor(np.random.randn(2, 5, 8).astype(np.float32)))[0].shape == (2, 4)
    assert dec.draft(vn.Tensor(np.random.randn(2, 1, 8).astype(np.float32)))[0].shape == (2, 4)
    assert dec.draft(np.random.randn(1, 8).astype(np.float32))[0].shape == (1, 4)


def test_draft_k_other_than_4(vn):
    for k in (2, 8):
        dec = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=k)
        t, lg = dec.draft(vn.Tensor(np.random.randn(1, 1, 8).astype(np.float32)))
        assert t.shape == (1, k) and len(lg) == k


def test_draft_head_invalid_k(vn):
    with pytest.raises(ValueError):
        vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=0)
    with pytest.raises(ValueError):
        vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=-1)


# ---- tests/test_speculative_decode.py:140-309 -----------------------------------------------------------------
def _draft_for(vn, dec, model, context):
    with vn.no_grad():
        hidden = model(vn.Tensor(context))[1]
    return dec.draft(hidden)[0]


def test_verify_accept_all(vn):
    model = ControlledMainModel(vn, next_token_logits=_table([10, 11, 12, 13]))
    dec = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=4)
    _force_heads(vn, dec, [10, 11, 12, 13])
    context = np.array([[1, 2, 3]], dtype=np.int64)
    draft = _draft_for(vn, dec, model, context)
    assert draft[0].tolist() == [10, 11, 12, 13]
    tokens, all_ok, _ = dec.verify_then_commit(draft, model, context)
    assert all_ok is True and tokens == [10, 11, 12, 13]


def test_verify_accept_partial_prefix(vn):
    model = ControlledMainModel(vn, next_token_logits=_table([10, 11, 12, 13]))
    dec = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=4)
    _force_heads(vn, dec, [10, 0, 0, 0])          # only the first proposal agrees with the target
    context = np.array([[1, 2, 3]], dtype=np.int64)
    draft = _draft_for(vn, dec, model, context)
    assert draft[0].tolist() == [10, 0, 0, 0]
    tokens, all_ok, _ = dec.verify_then_commit(draft, model, context, max_redraft_rounds=0)
    assert all_ok is False and tokens == [10, 11]


def test_verify_reject_first_position(vn):
    model = ControlledMainModel(vn, next_token_logits=_table([5, 6, 7, 8]))
    dec = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=4)
    _force_heads(vn, dec, [0, 1, 2, 3])
    context = np.array([[1, 2, 3]], dtype=np.int64)
    draft = _draft_for(vn, dec, model, context)
    assert draft[0].tolist() == [0, 1, 2, 3]
    tokens, all_ok, _ = dec.verify_then_commit(draft, model, context, max_redraft_rounds=0)
    assert all_ok is False and tokens == [5]


def test_verify_reject_triggers_redraft(vn):
    model = ControlledMainModel(vn, next_token_logits=_table([10, 11, 12, 13]))
    dec = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=4)
    _force_heads(vn, dec, [0, 1, 2, 3])
    context = np.array([[1, 2, 3]], dtype=np.int64)
    draft = _draft_for(vn, dec, model, context)
    tokens, all_ok, new_ctx = dec.verify_then_commit(draft, model, context, max_redraft_rounds=1)
    assert all_ok is False and tokens[0] == 10
    assert new_ctx.shape[1] == context.shape[1] + len(tokens)


# ---- tests/test_speculative_decode.py:317-409 -----------------------------------------------------------------
def test_full_draft_verify_pipeline(vn):
    V, D = 32, 16
    model = ControlledMainModel(vn, vocab_size=V, dim=D)
    dec = vn.SpeculativeDecoder(dim=D, vocab_size=V, num_draft_heads=4)
    context = np.array([[5, 6, 7, 8, 9]], dtype=np.int64)
    with vn.no_grad():
        hidden = model(vn.Tensor(context))[1]
    draft, _ = dec.draft(hidden)
    mask, pred = dec.verify(draft, model, context)
    assert mask.shape == (1, 4) and pred.shape == (1, 4) and mask.dtype == bool
    # what the mask and the predictions must be: the target's argmax at the positions the proposals sit on
    full = np.concatenate([context, draft], axis=1)
    want = np.argmax(model.E[full] @ model.W, axis=-1)[:, context.shape[1] - 1:context.shape[1] - 1 + 4]
    np.testing.assert_array_equal(pred, want)
    np.testing.assert_array_equal(mask, draft == want)
    tokens, all_ok, new_ctx = dec.verify_then_commit(draft, model, context)
    assert isinstance(tokens, list) and 1 <= len(tokens) <= 4 and isinstance(all_ok, bool)
    assert new_ctx.shape == (1, context.shape[1] + len(tokens))


def test_draft_loss_for_training(vn):
    V, D = 16, 8
    dec = vn.SpeculativeDecoder(dim=D, vocab_size=V, num_draft_heads=4)
    hidden = vn.Tensor(np.random.randn(2, 1, D).astype(np.float32), requires_grad=False)
    _, logits = dec.draft(hidden)
    target = np.random.randint(0, V, size=(2, 4))
    loss = dec.draft_loss(logits, target)
    assert loss.data.shape == () and float(loss.data) > 0
    loss.backward()
    for head in dec.draft_heads:
        assert head.weight.grad is not None and head.weight.grad.shape == (V, D)
    # the value is the mean cross-entropy of the heads' logits
    ce = 0.0
    for i, lg in enumerate(logits):
        x = np.asarray(lg, dtype=np.float64)
        lse = np.log(np.exp(x - x.max(-1, keepdims=True)).sum(-1)) + x.max(-1)
        ce += np.mean(lse - x[np.arange(2), target[:, i]])
    assert abs(float(loss) - ce / 4) < 1e-5


def test_verify_batch_mismatch_raises(vn):
    dec = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=4)
    draft = np.array([[1, 2, 3, 4]], dtype=np.int64)
    context = np.array([[1, 2], [3, 4]], dtype=np.int64)
    with pytest.raises(ValueError):
        dec.verify(draft, lambda x: vn.Tensor(np.zeros((1, 4, 16))), context)


def test_verify_main_model_returns_tuple_or_tensor(vn):
    V, D = 16, 8

    class TensorOnly:
        def __call__(self, idx):
            B, T = idx.data.shape
            return vn.Tensor(np.random.randn(B, T, V).astype(np.float32))

    class WithHidden:
        def __call__(self, idx):
            B, T = idx.data.shape
            return (vn.Tensor(np.random.randn(B, T, V).astype(np.float32)),
                    vn.Tensor(np.random.randn(B, T, D).astype(np.float32)))

    dec = vn.SpeculativeDecoder(dim=D, vocab_size=V, num_draft_heads=4)
    context = np.array([[1, 2, 3]], dtype=np.int64)
    draft = np.array([[5, 6, 7, 8]], dtype=np.int64)
    for m in (TensorOnly(), WithHidden()):
        acc, pred = dec.verify(draft, m, context)
        assert acc.shape == (1, 4) and pred.shape == (1, 4)


# ---- tests/test_device_backend.py:56-145: the operator block, on the "cuda" backend -----------------------------
@pytest.fixture()
def backend(vn):
    np.random.seed(42)
    vn.clear_backend_cache()
    return vn.get_backend("cuda")


def test_backend_device_type(backend):
    assert backend.device_type == "cuda"


def test_backend_matmul(backend):
    a = np.random.randn(2, 3).astype(np.float32)
    b = np.random.randn(3, 4).astype(np.float32)
    out = backend.matmul(a, b)
    assert out.shape == (2, 4)
    np.testing.assert_allclose(np.asarray(out), a @ b, atol=1e-5)


def test_backend_linear_with_and_without_bias(backend):
    x = np.random.randn(4, 3).astype(np.float32)
    w = np.random.randn(2, 3).astype(np.float32)
    b = np.random.randn(2).astype(np.float32)
    np.testing.assert_allclose(np.asarray(backend.linear(x, w, b)), x @ w.T + b, atol=1e-5)
    np.testing.assert_allclose(np.asarray(backend.linear(x, w, None)), x @ w.T, atol=1e-5)


def test_backend_softmax(backend):
    x = np.random.randn(3, 5).astype(np.float32)
    out = np.asarray(backend.softmax(x, dim=-1))
    np.testing.assert_allclose(out.sum(axis=-1), 1.0, atol=1e-6)
    big = np.asarray(backend.softmax(np.array([[1000.0, 1001.0, 1002.0]], dtype=np.float32), dim=-1))
    assert np.all(np.isfinite(big))


def test_backend_layernorm(backend):
    x = np.random.randn(4, 8).astype(np.float32)
    out = np.asarray(backend.layernorm(x, np.ones(8, np.float32), np.zeros(8, np.float32), eps=1e-5))
    np.testing.assert_allclose(out.mean(axis=-1), 0.0, atol=1e-4)
    out2 = np.asarray(backend.layernorm(x, np.full(8, 2.0, np.float32), np.full(8, 1.0, np.float32), eps=1e-5))
    np.testing.assert_allclose(out2.var(axis=-1), 4.0, atol=0.1)


def test_backend_rmsnorm(backend):
    x = np.random.randn(4, 8).astype(np.float32)
    out = np.asarray(backend.rmsnorm(x, np.ones(8, np.float32), eps=1e-6))
    np.testing.assert_allclose(np.sqrt((out * out).mean(axis=-1)), 1.0, atol=1e-4)


def test_backend_rope(backend):
    x = np.random.randn(2, 4, 8).astype(np.float32)
    np.testing.assert_allclose(np.asarray(backend.rope(x)), x)
    half = 4
    cos = np.random.randn(2, 4, half).astype(np.float32)
    sin = np.random.randn(2, 4, half).astype(np.float32)
    out = backend.rope(x, cos=cos, sin=sin)
    assert out.shape == x.shape
    x1, x2 = x[..., :half], x[..., half:]
    np.testing.assert_allclose(np.asarray(out), np.concatenate([x1 * cos - x2 * sin, x1 * sin + x2 * cos], -1),
                               atol=1e-5)


def test_backend_attention(backend):
    q, k, v = (np.random.randn(2, 4, 8).astype(np.float32) for _ in range(3))
    out = backend.attention(q, k, v)
    assert out.shape == (2, 4, 8)
    s = np.einsum("btd,bsd->bts", q, k) / np.sqrt(8.0)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    np.testing.assert_allclose(np.asarray(out), np.einsum("bts,bsd->btd", p, v), atol=1e-5)


def test_backend_factory_is_cached_by_lowercased_name(vn):
    vn.clear_backend_cache()
    a, b = vn.get_backend("cuda"), vn.get_backend("CUDA")
    assert a is b
    assert vn.get_backend("cuda:0") is vn.get_backend("cuda:0")
    with pytest.raises(RuntimeError):
        vn.get_backend("npu")
