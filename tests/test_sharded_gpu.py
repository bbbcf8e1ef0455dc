"""Vocabulary-sharded acceptance with the per-shard arithmetic on the device (`vn_row_stats`, `vn_row_residual`,
`vn_row_pick`): one GPU stands in for the ranks, every shard's logits live in their own device buffers, and the
three exchanges of the protocol are done by stacking the shards' small result arrays.  The outcome must equal the
unsharded rule of the CPU oracle on the concatenated logits."""

import numpy as np
import pytest

from oracle import accept as OA

pytestmark = pytest.mark.gpu


def _inputs(B, k, V, seed):
    rng = np.random.default_rng(seed)
    q = rng.normal(0, 2, (B, k, V)).astype(np.float32)
    p = np.concatenate([q + rng.normal(0, 0.5, (B, k, V)).astype(np.float32),
                        rng.normal(0, 2, (B, 1, V)).astype(np.float32)], axis=1)
    draft = np.argmax(q + rng.gumbel(size=q.shape), -1).astype(np.int64)
    return p, q, draft, rng.random((B, k)).astype(np.float32), rng.random((B, k + 1)).astype(np.float32)


@pytest.mark.parametrize("world,V,T,with_q", [(3, 1003, 1.0, True), (2, 9000, 0.7, True), (4, 40000, 1.0, False),
                                              (3, 1003, 0.0, True), (8, 248320, 1.0, True)])
def test_device_shards_match_unsharded_oracle(world, V, T, with_q):
    import versenext_b200 as vn
    from versenext_b200 import dist as vd
    from versenext_b200.sharded import DeviceShardOps, ShardedAccept, run_emulated
    ctx = vn.Context.get(0)
    B, k = (4, 4) if V > 100000 else (7, 4)
    p, q, draft, ua, us = _inputs(B, k, V, seed=V + world)
    parts = []
    for r in range(world):
        lo, hi = vd.vocab_shard(V, world, r, align=128 if V > 100000 else 8)
        pd = ctx.from_numpy(np.ascontiguousarray(p[..., lo:hi]))
        qd = ctx.from_numpy(np.ascontiguousarray(q[..., lo:hi])) if with_q else None
        parts.append(ShardedAccept(DeviceShardOps(ctx, pd, qd, T), draft, ua, us, lo, r, T))
    want_n, want_t = OA.accept(p, q if with_q else None, draft, ua, us, T, 0)
    for n, t in run_emulated(parts):
        np.testing.assert_array_equal(n, want_n)
        np.testing.assert_array_equal(t, want_t)


def test_row_stats_against_numpy():
    import ctypes as C
    import versenext_b200 as vn
    ctx = vn.Context.get(0)
    rng = np.random.default_rng(2)
    R, V = 11, 12345
    x = rng.normal(0, 3, (R, V)).astype(np.float32)
    x[3, :] = -np.inf                                  # a fully masked row
    tok = rng.integers(-1, V + 1, R).astype(np.int64)
    xd, td = ctx.from_numpy(x), ctx.from_numpy(tok)
    m, s, lx = ctx.empty((R,), np.float32), ctx.empty((R,), np.float64), ctx.empty((R,), np.float32)
    ptr = lambda a: C.c_void_p(a.ptr)
    ctx._check(ctx.lib.vn_row_stats(ctx.handle, ptr(xd), V, R, V, 0.5, ptr(td), ptr(m), ptr(s), ptr(lx)))
    xs = (x / np.float32(0.5)).astype(np.float32)
    wm = xs.max(axis=1)
    with np.errstate(invalid="ignore"):
        ws = np.where(np.isneginf(wm), 0.0, np.exp(xs - wm[:, None]).astype(np.float32).sum(axis=1, dtype=np.float64))
    np.testing.assert_array_equal(m.numpy(), wm)
    # 16 exponentials are added in float32 per thread before the float64 sums, chunk maxima are rescaled afterwards
    np.testing.assert_allclose(s.numpy(), ws, rtol=1e-6)
    inside = (tok >= 0) & (tok < V)
    wl = np.where(inside, xs[np.arange(R), np.clip(tok, 0, V - 1)], -np.inf)
    np.testing.assert_array_equal(lx.numpy(), wl.astype(np.float32))


def _nccl_worker(rank, world, port, out):
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    import versenext_b200 as vn
    from versenext_b200 import dist as vd
    from versenext_b200.sharded import DeviceShardOps, ShardedAccept, run_distributed
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = vn.Context.get(rank)
        B, k, V, T = 6, 4, 20000, 0.9
        p, q, draft, ua, us = _inputs(B, k, V, seed=77)
        lo, hi = vd.vocab_shard(V, world, rank, align=128)
        ops = DeviceShardOps(ctx, ctx.from_numpy(np.ascontiguousarray(p[..., lo:hi])),
                             ctx.from_numpy(np.ascontiguousarray(q[..., lo:hi])), T)
        n, t = run_distributed(ShardedAccept(ops, draft, ua, us, lo, rank, T))
        out.put((rank, n, t))
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_nccl():
    """The same protocol with one process per GPU and NCCL all-gathers (needs two GPUs; skipped on one)."""
    import socket
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    qout = ctx.Queue()
    procs = [ctx.Process(target=_nccl_worker, args=(r, 2, port, qout)) for r in range(2)]
    for pr in procs:
        pr.start()
    got = [qout.get(timeout=300) for _ in procs]
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    p, q, draft, ua, us = _inputs(6, 4, 20000, seed=77)
    want_n, want_t = OA.accept(p, q, draft, ua, us, 0.9, 0)
    for _, n, t in got:
        np.testing.assert_array_equal(n, want_n)
        np.testing.assert_array_equal(t, want_t)


def test_sharded_head_and_acceptance_from_hidden_states():
    """The data flow of a head split by columns: final-norm hidden rows -> each shard's logits (`vn_model_head`) ->
    the three-exchange acceptance.  Against the unsharded path on the same model: full logits from the forward,
    acceptance by `vn_accept` with the same injected uniforms."""
    import versenext_b200 as vn
    from oracle import model as OM
    from versenext_b200 import dist as vd, sampling
    from versenext_b200.sharded import DeviceShardOps, ShardedAccept, run_emulated
    ctx = vn.Context.get(0)
    models = []
    for seed in (41, 42):                                   # target, draft: same shape, different weights
        cfg = OM.mate_config(vocab_size=1024, dim=256, n_layer=2, n_head=4, n_kv_head=2, window_size=24,
                             num_global_tokens=20, max_seq_len=256, init_std=0.05, num_dense_parts=2,
                             num_experts_per_part=2, top_k=1)
        sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=seed, gate_std=1.0).items()}
        kw = cfg.to_dict()
        kw.pop("init_std")
        m = vn.VerseNexLM(dtype="bf16", **kw)
        m.load_state_dict(sd)
        models.append(m)
    target, draft_model = models
    rng = np.random.default_rng(12)
    B, k, V, T = 5, 4, 1024, 0.8
    toks = rng.integers(0, V, (B, 30 + k + 1))
    full, hid = [], []
    for m in models:
        cache = m.new_cache(B, 64)
        m.forward_cached(toks[:, :30], cache, last_only=True)
        cache.commit(30, np.full(B, 30, np.int32))
        lg, hd = m.forward_cached(toks[:, 30:], cache, want_hidden=True)
        full.append(lg)
        hid.append(hd)
    p_full = full[0].numpy()                                # [B, k+1, V]
    q_full = full[1].numpy()[:, :k]
    draft = np.argmax(q_full + rng.gumbel(size=q_full.shape), -1).astype(np.int64)
    ua = rng.random((B, k)).astype(np.float32)
    us = rng.random((B, k + 1)).astype(np.float32)
    want_n, want_t = sampling.accept(ctx, p_full, q_full, draft, u_accept=ua, u_sample=us, temperature=T)
    want_n, want_t = want_n.numpy(), want_t.numpy()
    world = 3
    parts = []
    for r in range(world):
        lo, hi = vd.vocab_shard(V, world, r, align=128)
        ps = target.head_columns(hid[0], lo, hi - lo)       # [B * (k+1), hi - lo]
        np.testing.assert_allclose(ps.numpy().reshape(B, k + 1, hi - lo), p_full[..., lo:hi], rtol=0, atol=1e-5)
        qs_all = draft_model.head_columns(hid[1], lo, hi - lo).numpy().reshape(B, k + 1, hi - lo)[:, :k]
        qs = ctx.from_numpy(np.ascontiguousarray(qs_all))
        ops = DeviceShardOps(ctx, ps.reshape(B, k + 1, hi - lo), qs, T)
        parts.append(ShardedAccept(ops, draft, ua, us, lo, r, T))
    for n, t in run_emulated(parts):
        np.testing.assert_array_equal(n, want_n)
        np.testing.assert_array_equal(t, want_t)
    target.check()


def _small_pair(vn, OM, vocab=1024):
    out = []
    for seed, n_layer in ((51, 2), (52, 1)):                # target, draft
        cfg = OM.mate_config(vocab_size=vocab, dim=256, n_layer=n_layer, n_head=4, n_kv_head=2, window_size=24,
                             num_global_tokens=20, max_seq_len=256, init_std=0.05, num_dense_parts=2,
                             num_experts_per_part=2, top_k=1)
        sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=seed, gate_std=1.0).items()}
        kw = cfg.to_dict()
        kw.pop("init_std")
        m = vn.VerseNexLM(dtype="bf16", **kw)
        m.load_state_dict(sd)
        out.append(m)
    return out


def _engine_tokens(eng, prompts, rounds):
    eng.prefill(prompts)
    for _ in range(rounds):
        eng.step()
    c = eng.counts()
    h = eng.history.numpy()
    return [h[b, :c[b]].copy() for b in range(len(c))]


def test_sharded_engine_equals_plain_engine_on_one_rank():
    """With one rank the column-split round (hidden rows -> head columns -> exchanges) must commit exactly the tokens
    of the plain engine: same Philox streams, same acceptance rule."""
    import versenext_b200 as vn
    from oracle import model as OM
    from versenext_b200.sharded_engine import ShardedSpecEngine
    target, draft = _small_pair(vn, OM)
    prompts = np.random.default_rng(13).integers(0, 1024, (6, 20))
    kw = dict(max_batch=6, max_seq=128, k=3, temperature=0.9, seed=17)
    plain = _engine_tokens(vn.SpecEngine(target, draft, top_k=0, graph=False, **kw), prompts, 6)
    shard = _engine_tokens(ShardedSpecEngine(target, draft, **kw), prompts, 6)
    for a, b in zip(plain, shard):
        np.testing.assert_array_equal(a, b)
    assert sum(len(a) for a in plain) > 6 * 6               # some proposals were accepted


@pytest.mark.parametrize("scheme", ["int8", "int4g128"])
def test_sharded_engine_with_a_quantised_target(scheme):
    """Vocabulary-sharded acceptance on a weight-only quantised target (the INT8 / INT4 variants of the sharded
    configuration): the column-split head works on the quantised head copy, and the round commits the tokens of
    the plain engine run on the same quantised models."""
    import versenext_b200 as vn
    from oracle import model as OM
    from versenext_b200.sharded_engine import ShardedSpecEngine
    target, draft = _small_pair(vn, OM)
    target.quantize(scheme)
    prompts = np.random.default_rng(14).integers(0, 1024, (6, 20))
    kw = dict(max_batch=6, max_seq=128, k=3, temperature=0.9, seed=19)
    plain = _engine_tokens(vn.SpecEngine(target, draft, top_k=0, graph=False, **kw), prompts, 6)
    shard = _engine_tokens(ShardedSpecEngine(target, draft, **kw), prompts, 6)
    for a, b in zip(plain, shard):
        np.testing.assert_array_equal(a, b)
    target.check()


def _engine_worker(rank, world, port, out):
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    import versenext_b200 as vn
    from oracle import model as OM
    from versenext_b200.sharded_engine import ShardedSpecEngine
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = vn.Context.get(rank)
        cfgs = []
        models = []
        for seed, n_layer in ((51, 2), (52, 1)):
            cfg = OM.mate_config(vocab_size=1024, dim=256, n_layer=n_layer, n_head=4, n_kv_head=2, window_size=24,
                                 num_global_tokens=20, max_seq_len=256, init_std=0.05, num_dense_parts=2,
                                 num_experts_per_part=2, top_k=1)
            sd = {n: OM.bf16_round(v) for n, v in OM.init_state_dict(cfg, seed=seed, gate_std=1.0).items()}
            kw = cfg.to_dict()
            kw.pop("init_std")
            m = vn.VerseNexLM(dtype="bf16", device=f"cuda:{rank}", **kw)
            m.load_state_dict(sd)
            models.append(m)
        prompts = np.random.default_rng(100 + rank).integers(0, 1024, (4, 20))
        from versenext_b200.comm import Comm
        from versenext_b200.sharded_engine import rank_seed
        comm = Comm.from_torch_group(ctx)
        kw = dict(max_batch=4, max_seq=128, k=3, temperature=0.9)
        # the plain engine of this rank draws with the seed the sharded engine gives this rank's requests
        plain = _engine_tokens(vn.SpecEngine(models[0], models[1], top_k=0, graph=False, seed=rank_seed(17, rank), **kw),
                               prompts, 5)
        shard = _engine_tokens(ShardedSpecEngine(models[0], models[1], seed=17, comm=comm, **kw), prompts, 5)
        out.put((rank, all(np.array_equal(a, b) for a, b in zip(plain, shard)), sum(len(a) for a in plain)))
    finally:
        dist.destroy_process_group()


def test_sharded_engine_two_ranks_over_nccl():
    """Two processes, two GPUs: requests split over the ranks and the head split by columns, hidden rows and per-row
    statistics exchanged by the library's own NCCL all-gathers, decisions taken on the device; every rank commits
    the tokens its plain single-GPU engine commits for the same requests (needs two GPUs; skipped on one)."""
    import socket
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    qout = ctx.Queue()
    procs = [ctx.Process(target=_engine_worker, args=(r, 2, port, qout)) for r in range(2)]
    for pr in procs:
        pr.start()
    got = [qout.get(timeout=300) for _ in procs]
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    for rank, same, n in got:
        assert same, f"rank {rank}: sharded round differs from the plain engine"
        assert n > 0
