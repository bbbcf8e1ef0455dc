"""`vn_accept_noalloc`: the acceptance entry point for hosts that cannot allocate device memory.

A serving process that has handed the whole GPU to its own memory pool, or a framework that forbids
cudaMalloc once it is running, cannot let `vn_accept` grow its scratch buffer.  The no-alloc variant
keeps that scratch in a fixed array inside the library, so it must give exactly the results of
`vn_accept` -- bit for bit, since both run the same integer / float64 decision arithmetic -- on every
call, including a second call that finds the first call's leftovers in the shared array.

This file sorts last on purpose: a run that stops at the first failure has then already run every other
test.  It passes alone in a fresh process as well as after the rest of the suite.
"""

import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ptr(a):
    return C.c_void_p(a.ptr) if a is not None else C.c_void_p(None)


def _inputs(rng, B, k, V):
    q = rng.normal(0, 2.0, (B, k, V)).astype(np.float32)
    p = np.empty((B, k + 1, V), np.float32)
    p[:, :k] = q + rng.normal(0, 0.5, (B, k, V)).astype(np.float32)
    p[:, k] = rng.normal(0, 2.0, (B, V)).astype(np.float32)
    draft = np.argmax(q + rng.gumbel(size=q.shape), axis=-1).astype(np.int64)
    return p, q, draft


def _run(ctx, fn_name, p, q, draft, seed, offset, temperature, bonus=1):
    """Call one of the two entry points straight through the C ABI."""
    B, k = draft.shape
    V = p.shape[-1]
    out_len = ctx.zeros((B,), np.int32)
    out_tok = ctx.zeros((B, k + 1), np.int64)
    lib = ctx.lib
    if fn_name == "vn_accept":
        st = lib.vn_accept(ctx.handle, _ptr(p), _ptr(q), _ptr(draft), None, None, seed, offset, temperature,
                           0, bonus, B, k, V, _ptr(out_len), _ptr(out_tok))
    else:
        st = lib.vn_accept_noalloc(ctx.handle, _ptr(p), _ptr(q), _ptr(draft), None, None, seed, offset,
                                   temperature, bonus, B, k, V, _ptr(out_len), _ptr(out_tok))
    ctx._check(st)
    return out_len.numpy(), out_tok.numpy()


def test_noalloc_matches_allocating_entry_point_twice_in_a_row():
    import versenext_b200 as vn
    ctx = vn.Context.get(0)
    rng = np.random.default_rng(2024)
    # two different problems back to back: the second call sees the first call's data in the shared scratch
    for call, (B, k, V, temperature) in enumerate([(12, 4, 50000, 1.0), (7, 3, 8195, 0.7)]):
        p, q, draft = _inputs(rng, B, k, V)
        pd, qd, dd = ctx.from_numpy(p), ctx.from_numpy(q), ctx.from_numpy(draft)
        want_len, want_tok = _run(ctx, "vn_accept", pd, qd, dd, 99, call, temperature)
        got_len, got_tok = _run(ctx, "vn_accept_noalloc", pd, qd, dd, 99, call, temperature)
        np.testing.assert_array_equal(got_len, want_len)
        np.testing.assert_array_equal(got_tok, want_tok)
        assert np.all(got_tok[np.arange(B), got_len] >= 0)
    # greedy rule through the same entry point, again right after a stochastic call
    p, q, draft = _inputs(rng, 5, 4, 12345)
    draft[0] = np.argmax(p[0, :4], -1)
    pd, dd = ctx.from_numpy(p), ctx.from_numpy(draft)
    want = _run(ctx, "vn_accept", pd, None, dd, 0, 0, 0.0)
    got = _run(ctx, "vn_accept_noalloc", pd, None, dd, 0, 0, 0.0)
    np.testing.assert_array_equal(got[0], want[0])
    np.testing.assert_array_equal(got[1], want[1])
    assert got[0][0] == 4


def test_noalloc_follows_the_device_round_counter_and_allocates_nothing():
    """With a round counter on the device (what a captured decode round uses) both entry points draw the same
    Philox numbers; and a warm call leaves the amount of free device memory where it was."""
    import versenext_b200 as vn
    ctx = vn.Context.get(0)
    rng = np.random.default_rng(7)
    p, q, draft = _inputs(rng, 9, 4, 20000)
    pd, qd, dd = ctx.from_numpy(p), ctx.from_numpy(q), ctx.from_numpy(draft)
    counter = ctx.from_numpy(np.array([5], np.uint32))
    base = _run(ctx, "vn_accept", pd, qd, dd, 31, 0, 1.0)
    ctx._check(ctx.lib.vn_set_offset_source(ctx.handle, _ptr(counter)))
    try:
        want = _run(ctx, "vn_accept", pd, qd, dd, 31, 0, 1.0)
        got = _run(ctx, "vn_accept_noalloc", pd, qd, dd, 31, 0, 1.0)
    finally:
        ctx._check(ctx.lib.vn_set_offset_source(ctx.handle, None))
    np.testing.assert_array_equal(got[0], want[0])
    np.testing.assert_array_equal(got[1], want[1])
    shifted = _run(ctx, "vn_accept_noalloc", pd, qd, dd, 31, 5, 1.0)      # the same offset given by the host
    np.testing.assert_array_equal(shifted[1], got[1])
    assert not np.array_equal(base[1], got[1])                            # the counter really moved the streams
    # nothing allocated: outputs come from the caller, scratch from the library image
    out_len, out_tok = ctx.zeros((9,), np.int32), ctx.zeros((9, 5), np.int64)
    ctx.sync()
    free0, _ = ctx.mem_info()
    for _ in range(3):
        ctx._check(ctx.lib.vn_accept_noalloc(ctx.handle, _ptr(pd), _ptr(qd), _ptr(dd), None, None, 31, 0, 1.0, 1,
                                             9, 4, 20000, _ptr(out_len), _ptr(out_tok)))
    ctx.sync()
    free1, _ = ctx.mem_info()
    assert free1 == free0


def test_noalloc_rejects_sizes_beyond_its_scratch():
    import versenext_b200 as vn
    ctx = vn.Context.get(0)
    B, k, V = 256, 4, 248320           # needs about 2.5 MB of scratch: more than the built-in 2 MiB
    p = ctx.empty((1,), np.float32)    # never dereferenced: the size check comes first
    d = ctx.empty((1,), np.int64)
    out_len, out_tok = ctx.empty((B,), np.int32), ctx.empty((B, k + 1), np.int64)
    st = ctx.lib.vn_accept_noalloc(ctx.handle, _ptr(p), _ptr(p), _ptr(d), None, None, 1, 0, 1.0, 1, B, k, V,
                                   _ptr(out_len), _ptr(out_tok))
    assert st == 1  # VN_ERR_INVALID
    msg = ctx.lib.vn_last_error(ctx.handle).decode()
    assert "scratch" in msg and "vn_accept" in msg
    with pytest.raises(ValueError):
        ctx._check(st)
