"""SpeculativeDecoder drop-in against the outcomes recorded from the reference class."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


class TableModel:
    def __init__(self, table, as_tuple=False, dim=8):
        self.table, self.as_tuple, self.dim = table, as_tuple, dim

    def __call__(self, idx):
        import versenext_b200 as vn
        ids = np.asarray(idx.data)
        B, T = ids.shape
        lg = np.broadcast_to(self.table[None, :T], (B, T, self.table.shape[1])).astype(np.float32).copy()
        t = vn.Tensor(lg)
        return (t, vn.Tensor(np.zeros((B, T, self.dim), np.float32))) if self.as_tuple else t


def test_reference_recorded_cases(golden):
    import versenext_b200 as vn
    g = golden("spec_reference.npz")
    for ci in g["cases"]:
        p = f"c{ci}_"
        heads = g[p + "heads"]
        k, V, D = heads.shape
        dec = vn.SpeculativeDecoder(dim=D, vocab_size=V, num_draft_heads=k)
        for h, w in zip(dec.draft_heads, heads):
            h.weight.data = w
        draft, logits = dec.draft(vn.Tensor(g[p + "hidden"]))
        assert draft.dtype == np.int64 and draft.shape == g[p + "draft"].shape
        np.testing.assert_array_equal(draft, g[p + "draft"])
        assert len(logits) == k
        np.testing.assert_allclose(np.stack([np.asarray(l) for l in logits]), g[p + "draft_logits"],
                                   rtol=1e-5, atol=1e-5)
        model = TableModel(g[p + "table"], as_tuple=bool(ci % 2))
        mask, pred = dec.verify(g[p + "draft"], model, g[p + "ctx"])
        assert mask.dtype == bool
        np.testing.assert_array_equal(mask, g[p + "mask"])
        np.testing.assert_array_equal(pred, g[p + "pred"])
        toks, ok, new_ctx = dec.verify_then_commit(g[p + "draft"], model, g[p + "ctx"],
                                                   max_redraft_rounds=int(ci % 2))
        assert toks == [int(t) for t in g[p + "tokens"]]
        assert ok == bool(g[p + "all_ok"])
        np.testing.assert_array_equal(new_ctx, g[p + "new_ctx"])


def _forced(dec, tokens):
    for h, t in zip(dec.draft_heads, tokens):
        h.weight.data[:] = 0.0
        h.weight.data[t, :] = 10.0


def test_accept_all_partial_and_reject_first():
    """The three outcomes the reference's own tests pin: [10,11,12,13]/True, [10,11]/False, [5]/False."""
    import versenext_b200 as vn
    V, D, k = 16, 8, 4
    dec = vn.SpeculativeDecoder(dim=D, vocab_size=V, num_draft_heads=k)
    _forced(dec, [10, 11, 12, 13])
    hidden = np.ones((1, 1, D), np.float32)
    draft, _ = dec.draft(hidden)
    np.testing.assert_array_equal(draft, [[10, 11, 12, 13]])
    ctx_tok = np.array([[1, 2, 3]], np.int64)

    def table(seq):
        t = np.zeros((ctx_tok.shape[1] + k, V), np.float32)
        for i, tok in enumerate(seq):
            t[ctx_tok.shape[1] - 1 + i, tok] = 10.0
        return TableModel(t)

    toks, ok, new_ctx = dec.verify_then_commit(draft, table([10, 11, 12, 13]), ctx_tok)
    assert toks == [10, 11, 12, 13] and ok is True and new_ctx.shape == (1, 7)
    toks, ok, new_ctx = dec.verify_then_commit(draft, table([10, 11, 5, 13]), ctx_tok, max_redraft_rounds=0)
    assert toks == [10, 11, 5] and ok is False and new_ctx.shape == (1, 6)
    toks, ok, new_ctx = dec.verify_then_commit(draft, table([5, 11, 12, 13]), ctx_tok, max_redraft_rounds=0)
    assert toks == [5] and ok is False
    np.testing.assert_array_equal(new_ctx, [[1, 2, 3, 5]])


def test_hidden_shapes_k_values_and_errors():
    import versenext_b200 as vn
    rng = np.random.default_rng(0)
    dec = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=4)
    for shape in [(2, 8), (2, 5, 8), (2, 1, 8), (2, 3, 5, 8)]:
        t, lg = dec.draft(rng.normal(0, 1, shape).astype(np.float32))
        assert t.shape == (2, 4) and len(lg) == 4 and lg[0].shape == (2, 16)
        assert np.all((t >= 0) & (t < 16))
    with pytest.raises(ValueError):
        dec.draft(np.zeros((8,), np.float32))
    for k in (2, 8):
        d = vn.SpeculativeDecoder(dim=8, vocab_size=16, num_draft_heads=k)
        t, lg = d.draft(vn.Tensor(rng.normal(0, 1, (1, 1, 8)).astype(np.float32)))
        assert t.shape == (1, k) and len(lg) == k
    model = TableModel(np.zeros((20, 16), np.float32))
    with pytest.raises(ValueError):
        dec.verify(np.zeros((2, 4), np.int64), model, np.zeros((3, 5), np.int64))
    with pytest.raises(ValueError):
        dec.verify(np.zeros((4,), np.int64), model, np.zeros((1, 5), np.int64))


def test_batch_rows_beyond_zero_are_ignored_by_commit_and_served_by_commit_batch():
    import versenext_b200 as vn
    V, k = 16, 3
    dec = vn.SpeculativeDecoder(dim=8, vocab_size=V, num_draft_heads=k)
    t = np.zeros((6, V), np.float32)
    t[2, 4] = t[3, 5] = t[4, 6] = 9.0
    draft = np.array([[4, 5, 6], [4, 7, 6]], np.int64)
    ctx_tok = np.array([[1, 2, 3], [3, 2, 1]], np.int64)
    toks, ok, new_ctx = dec.verify_then_commit(draft, TableModel(t), ctx_tok)
    assert toks == [4, 5, 6] and ok and new_ctx.shape == (1, 6)
    rows, lens = dec.commit_batch(draft, TableModel(t), ctx_tok)
    np.testing.assert_array_equal(lens, [3, 1])
    np.testing.assert_array_equal(rows, [[4, 5, 6, -1], [4, 5, -1, -1]])
