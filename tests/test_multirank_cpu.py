"""World-size-2 checks of the multi-rank host logic on CPU (gloo): request sharding, the max-over-ranks
and sum reductions the benchmark uses, and the (max, sum-exp) exchange of a vocabulary-sharded head."""

import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import torch.distributed as dist
    from versenext_b200 import dist as vd
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        res = {}
        assert vd.env_world() == (world, rank, rank)
        lo, hi = vd.shard_range(33, world, rank)
        res["shard"] = (lo, hi)
        res["max"] = vd.reduce_max(10.0 + rank)
        res["sum"] = vd.reduce_sum(float(hi - lo))
        # vocabulary-sharded softmax statistics of 5 rows over V = 1000
        rng = np.random.default_rng(0)
        logits = rng.normal(0, 3, (5, 1000))
        vlo, vhi = vd.vocab_shard(1000, world, rank, align=8)
        part = logits[:, vlo:vhi]
        lm = part.max(axis=1)
        ls = np.exp(part - lm[:, None]).sum(axis=1)
        gm, gs = vd.combine_softmax_partials(lm, ls)
        res["gm"], res["gs"] = gm, gs
        res["vshard"] = (vlo, vhi)
        out.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0]["shard"] == (0, 17) and got[1]["shard"] == (17, 33)
    assert got[0]["max"] == got[1]["max"] == 11.0
    assert got[0]["sum"] == got[1]["sum"] == 33.0
    assert got[0]["vshard"][1] == got[1]["vshard"][0] and got[1]["vshard"][1] == 1000
    logits = np.random.default_rng(0).normal(0, 3, (5, 1000))
    m = logits.max(axis=1)
    s = np.exp(logits - m[:, None]).sum(axis=1)
    for r in (0, 1):
        np.testing.assert_allclose(got[r]["gm"], m)
        np.testing.assert_allclose(got[r]["gs"], s, rtol=1e-12)


def _accept_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import torch.distributed as dist
    from versenext_b200 import dist as vd
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        res = {}
        for name, (p, q, draft, ua, us, T) in _accept_cases().items():
            V = p.shape[-1]
            lo, hi = vd.vocab_shard(V, world, rank, align=8)
            qs = None if q is None else q[..., lo:hi]
            res[name] = vd.sharded_accept(p[..., lo:hi], qs, draft, ua, us, lo, T)
        out.put((rank, res))
    finally:
        dist.destroy_process_group()


def _accept_cases():
    rng = np.random.default_rng(11)
    B, k, V = 7, 4, 1003
    q = rng.normal(0, 2, (B, k, V)).astype(np.float32)
    p = np.concatenate([q + rng.normal(0, 0.5, (B, k, V)).astype(np.float32),
                        rng.normal(0, 2, (B, 1, V)).astype(np.float32)], axis=1)
    draft = np.argmax(q + rng.gumbel(size=q.shape), -1).astype(np.int64)
    ua = rng.random((B, k)).astype(np.float32)
    us = rng.random((B, k + 1)).astype(np.float32)
    small = (p[:, :, :20].copy(), q[:, :, :20].copy(), draft % 20, ua, us, 1.0)   # 20 columns: an empty last shard
    return {"t1": (p, q, draft, ua, us, 1.0), "t07": (p, q, draft, ua, us, 0.7), "greedy": (p, q, draft, ua, us, 0.0),
            "point_mass": (p, None, draft, ua, us, 1.0), "tiny": small}


@pytest.mark.parametrize("world", [2, 3])
def test_vocabulary_sharded_acceptance_matches_unsharded_rule(world):
    """The exchange protocol of the sharded LM head + acceptance (stats and token logits, residual masses, picked
    token) on gloo ranks: every rank returns the decisions and tokens of the unsharded rule."""
    import torch.multiprocessing as mp
    from oracle import accept as OA
    ctx = mp.get_context("spawn")
    qout = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_accept_worker, args=(r, world, port, qout)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(qout.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for name, (pl, ql, draft, ua, us, T) in _accept_cases().items():
        want_n, want_t = OA.accept(pl, ql, draft, ua, us, T, 0)
        for r in range(world):
            n, t = got[r][name]
            np.testing.assert_array_equal(n, want_n, err_msg=f"{name} rank {r}")
            np.testing.assert_array_equal(t, want_t, err_msg=f"{name} rank {r}")


def test_shard_helpers_single_process():
    from versenext_b200 import dist as vd
    for total in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            spans = [vd.shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
    with pytest.raises(ValueError):
        vd.shard_range(4, 2, 2)
    spans = [vd.vocab_shard(248320, 8, r) for r in range(8)]
    assert spans[0] == (0, 31104) and spans[-1][1] == 248320 and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert vd.reduce_max(3.0) == 3.0 and vd.reduce_sum(2.0) == 2.0
    m, s = vd.merge_softmax_partials(np.array([[1.0, -np.inf], [0.0, 2.0]]), np.array([[2.0, 0.0], [1.0, 3.0]]))
    np.testing.assert_allclose(m, [1.0, 2.0])
    np.testing.assert_allclose(s, [2.0 + np.exp(-1.0), 3.0])
