#!/usr/bin/env python
"""Benchmark of the speculative-decoding hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload spec|accept]

Prints ONE JSON line (rank 0).  Workloads:

  spec     (default) full speculative decode: mate-shaped VerseNexLM target (dim 1024, 20 layers =
           5 MoD + 15 TriSparse, vocab 248320, bf16, tied head, seeded N(0, 0.02) weights) with a
           2-layer dim-256 draft over the same vocabulary, k=4, temperature 0.8, top-k 50, 32
           requests per GPU with 512-token uniform-random prompts.  A step is one round
           (draft 4 tokens -> verify 5 positions -> accept -> commit) over the whole batch;
           metric = accepted tok/s = tokens committed / time.  Prefill is outside the timed region.

  accept   isolated acceptance-sampling op: B=64 sequences, k=4 draft positions,
           vocab 248320, fp32 target logits [B,k+1,V] and draft logits [B,k,V]
           (draft ~ N(0, 2^2), target = draft + N(0, 0.5^2)), temperature 1,
           Philox uniforms seed 1234.  metric = sampler GB/s over the
           572,129,280 logit bytes every call has to read once.

A step is one pass of the op over one batch.  With N > 1 every rank owns its
own batch of requests (no data-path collective): weak scaling.
`--impl reference` times the CPU restatement of the reference's algorithm
(oracle/, NumPy, one host thread) on a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

if "reference" in sys.argv[1:] or "--impl=reference" in sys.argv[1:]:
    # The CPU arm uses every host core.  BLAS reads these variables when NumPy loads it, so they are set before
    # the import below; torchrun exports OMP_NUM_THREADS=1 to its workers, which is overridden here on purpose.
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(os.cpu_count() or 1)

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ACCEPT = dict(B=64, k=4, V=248320, seed=1234, temperature=1.0)


# DRAM bytes of one verify + accept step of the default workload, summed over its kernels from the ncu capture
# summarised in profiles/spec_step_dram_traffic.txt (B=32, ctx about 550).  ncu flushes the caches before every
# kernel, so partial tiles and logits that the real run finds in L2 count as DRAM here: an upper bound.
SPEC_STEP_TRAFFIC = 3565000000


def accept_bytes(B, k, V):
    return B * (k + 1) * V * 4 + B * k * V * 4


def make_accept_inputs(B, k, V, seed):
    """Seeded synthetic logits of the acceptance workload (float32)."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, k, V), dtype=np.float32) * np.float32(2.0)
    p = np.empty((B, k + 1, V), dtype=np.float32)
    p[:, :k] = q + rng.standard_normal((B, k, V), dtype=np.float32) * np.float32(0.5)
    p[:, k] = rng.standard_normal((B, V), dtype=np.float32) * np.float32(2.0)
    # draft tokens distributed as softmax(q): Gumbel-max
    draft = np.empty((B, k), dtype=np.int64)
    for b in range(B):
        g = rng.gumbel(size=(k, V)).astype(np.float32)
        draft[b] = np.argmax(q[b] + g, axis=-1)
    return p, q, draft


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def blas_threads():
    """Threads the BLAS behind NumPy really uses (threadpoolctl), else the environment's request."""
    try:
        from threadpoolctl import threadpool_info
        n = [int(d.get("num_threads", 0)) for d in threadpool_info() if d.get("user_api") == "blas"]
        if n:
            return max(n)
    except Exception:
        pass
    return int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))


def timed_repeats(run_k_steps, prepare, ctx, dist, local, min_repeats=5, min_total_ms=1000.0, max_repeats=40):
    """`prepare()` (untimed) then K steps between two CUDA events on the context's stream, bracketed by a
    barrier and a device synchronisation on both sides, repeated until at least `min_repeats` repeats and
    `min_total_ms` of timed work are in.  Every repeat's time is the maximum over the ranks.
    Returns the list of repeat times in ms."""
    reps = []
    while True:
        prepare()
        barrier_sync(dist, ctx)
        e0, e1 = ctx.event(), ctx.event()
        e0.record()
        run_k_steps()
        e1.record()
        ms = e0.elapsed_ms(e1)
        barrier_sync(dist, ctx)
        reps.append(max_over_ranks(dist, ms, local))
        if len(reps) >= min_repeats and (sum(reps) >= min_total_ms or len(reps) >= max_repeats):
            return reps


def spread(reps, steps):
    per = sorted(r / steps for r in reps)
    return {"repeats": len(per), "median_ms_per_step": statistics.median(per), "min_ms_per_step": per[0],
            "max_ms_per_step": per[-1], "timed_ms_total": sum(reps)}


def dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        # NCCL prints its version banner (and, at higher debug levels, more) to file descriptor 1 when the first
        # communicator comes up.  Stdout must carry the one JSON line only, so descriptor 1 points at stderr while
        # the process group and its first collective are set up.
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local)
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
            t = torch.zeros(1, device=f"cuda:{local}")
            dist_mod.all_reduce(t)
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
        dist = dist_mod
    return world, rank, local, dist


def barrier_sync(dist, ctx):
    ctx.sync()
    if dist is not None:
        import torch
        dist.barrier()
        torch.cuda.synchronize()


def max_over_ranks(dist, value, local):
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=f"cuda:{local}")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ---------------------------------------------------------------------------
# CPU baseline (oracle port)
# ---------------------------------------------------------------------------

def cpu_accept_sample(n_seq, repeats=1):
    """Time the NumPy restatement on `n_seq` sequences of the workload; returns (GB/s, seconds)."""
    from oracle import accept as OA
    from oracle import philox as OP
    k, V = ACCEPT["k"], ACCEPT["V"]
    p, q, draft = make_accept_inputs(n_seq, k, V, ACCEPT["seed"])
    ua, us = OP.uniforms_for_call(ACCEPT["seed"], 0, n_seq, k)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        OA.accept(p, q, draft, ua, us, ACCEPT["temperature"], 0)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return accept_bytes(n_seq, k, V) / best / 1e9, best


# ---------------------------------------------------------------------------
# speculative decode workload
# ---------------------------------------------------------------------------

SPEC = dict(B=32, prompt=512, k=4, temperature=0.8, top_k=50, seed=4, new_tokens=256)
SPEC_WORKLOAD = ("spec: mate target (D=1024, L=20: 5 MoD + 15 TriSparse, V=248320, bf16) + 2-layer D=256 draft, "
                 "k=4, T=0.8, top-k 50, 32 requests of 512-token prompts")
MATE_PARAMS = 1107375164


def spec_step_bytes(B, ctx_len, dtype_bytes=2):
    """Algorithmic bytes of one verify+sample step: every unique target weight once, plus the K/V window
    (20 layers x B x min(ctx, 1024) positions x (2 x 512) values)."""
    return MATE_PARAMS * dtype_bytes + 20 * B * min(ctx_len, 1024) * 2 * 512 * dtype_bytes


def spec_prompts(B, T, seed, rank=0):
    return np.random.default_rng([seed, rank]).integers(0, 248320, (B, T)).astype(np.int64)


def build_spec_models(device="cuda"):
    import versenext_b200 as vn
    from versenext_b200 import synthetic as S
    tk, dk = S.mate_kwargs(), S.draft_kwargs()
    target = vn.VerseNexLM(dtype="bf16", device=device, **tk)
    S.load_random(target, tk, seed=0)
    draft = vn.VerseNexLM(dtype="bf16", device=device, **dk)
    S.load_random(draft, dk, seed=1)
    return target, draft


def cpu_spec_sample(max_seconds=25.0, rounds=2, warmup=1):
    """Reference algorithm on the host (NumPy restatement, BLAS threads = all cores): one request of the
    workload, full re-forward of [context, draft] every round as the reference does.  Returns
    (tok/s, seconds, rounds run)."""
    from oracle import model as OM
    from oracle import spec as OS
    from versenext_b200 import synthetic as S
    tk, dk = S.mate_kwargs(), S.draft_kwargs()
    t_cfg = OM.mate_config()
    d_cfg = OM.Config(**{k: v for k, v in dk.items()})
    t_sd = dict(S.random_tensors(tk, seed=0))
    t_sd["head.weight"] = t_sd["tok_emb.weight"]
    d_sd = dict(S.random_tensors(dk, seed=1))
    d_sd["head.weight"] = d_sd["tok_emb.weight"]
    prompt = spec_prompts(1, SPEC["prompt"], SPEC["seed"])
    seq = prompt
    for _ in range(warmup):              # untimed: first-touch of the weights, BLAS thread start-up
        st = OS.generate(t_sd, t_cfg, d_sd, d_cfg, seq, SPEC["k"], 10 ** 6, temperature=SPEC["temperature"],
                         top_k=SPEC["top_k"], seed=SPEC["seed"], bonus=True, max_rounds=1)
        seq = st["tokens"][0]
    t0 = time.perf_counter()
    done = committed = 0
    while done < rounds and time.perf_counter() - t0 < max_seconds:
        st = OS.generate(t_sd, t_cfg, d_sd, d_cfg, seq, SPEC["k"], 10 ** 6, temperature=SPEC["temperature"],
                         top_k=SPEC["top_k"], seed=SPEC["seed"], bonus=True, max_rounds=1)
        new_seq = st["tokens"][0]
        committed += new_seq.shape[1] - seq.shape[1]
        seq = new_seq
        done += 1
    dt = time.perf_counter() - t0
    return committed / dt, dt, done


def _spec_engine(vn, target, draft, B, args, warm):
    k, T0 = SPEC["k"], SPEC["prompt"]
    rounds = warm + args.steps + 8
    return vn.SpecEngine(target, draft, max_batch=B, max_seq=T0 + rounds * (k + 1) + 64, k=k,
                         temperature=SPEC["temperature"], top_k=SPEC["top_k"], seed=SPEC["seed"], bonus=True,
                         max_new_tokens=rounds * (k + 1))


def _time_engine(eng, ctx, dist, local, steps, warm):
    """Rounds per second of one engine: every repeat starts from the state right after prefill (so the context
    length, and with it the K/V window that is read, is the same in every repeat), runs `warm` untimed rounds
    and then exactly `steps` timed ones.  Returns (repeat times ms, tokens committed in the timed rounds of the
    last repeat on this rank)."""
    box = {}

    def prepare():
        eng.rewind()
        for _ in range(warm):
            eng.step()
        box["c0"] = int(eng.counts().sum())

    def run():
        for _ in range(steps):
            eng.step()

    reps = timed_repeats(run, prepare, ctx, dist, local)
    return reps, int(eng.counts().sum()) - box["c0"]


def _sum_over_ranks(dist, value, local):
    if dist is None:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=f"cuda:{local}")
    dist.all_reduce(t)
    return float(t.item())


def _sharded_check(vn, target, draft, dist, ctx, local, world, rank, rounds=4):
    """Vocabulary-sharded head + acceptance over the ranks (the one data path with an exchange): a few rounds of
    the sharded engine on this rank's requests must commit exactly the tokens of its plain engine."""
    from versenext_b200.comm import Comm
    from versenext_b200.sharded_engine import ShardedSpecEngine, rank_seed
    B, k, T0 = 8, SPEC["k"], 64
    prompts = spec_prompts(B, T0, 99, rank)
    kw = dict(max_batch=B, max_seq=T0 + (rounds + 2) * (k + 1) + 16, k=k, temperature=1.0,
              max_new_tokens=(rounds + 2) * (k + 1))
    comm = Comm.from_torch_group(ctx) if dist is not None else None
    plain = vn.SpecEngine(target, draft, top_k=0, bonus=True, graph=False, seed=rank_seed(5, rank), **kw)
    plain.prefill(prompts)
    for _ in range(rounds):
        plain.step()
    want = plain.history.numpy()[:, :rounds]
    want_counts = plain.counts()
    del plain
    sh = ShardedSpecEngine(target, draft, seed=5, comm=comm, **kw)
    sh.prefill(prompts)
    sh.step()                                   # warm-up round (buffers, communicators)
    sh.rewind()
    barrier_sync(dist, ctx)
    t0 = time.perf_counter()
    for _ in range(rounds):
        sh.step()
    ctx.sync()
    ms = (time.perf_counter() - t0) * 1e3 / rounds
    ok = bool(np.array_equal(sh.counts(), want_counts) and np.array_equal(sh.history.numpy()[:, :rounds], want))
    ok_all = _sum_over_ranks(dist, 1.0 if ok else 0.0, local) == world
    return {"ok": bool(ok_all), "ms_per_round": max_over_ranks(dist, ms, local), "n_ranks": world,
            "requests_per_rank": B, "rounds": rounds,
            "what": "ShardedSpecEngine (LM head + acceptance split by vocabulary columns over the ranks, exchanges "
                    "as NCCL all-gathers of device buffers on the library's stream, no host synchronisation) commits "
                    "the same tokens as the plain engine on every rank"}


def run_spec(args):
    import versenext_b200 as vn
    world, rank, local, dist = dist_setup(args.gpus)
    ctx = vn.Context.get(local)
    k, T0 = SPEC["k"], SPEC["prompt"]
    # The configuration is 32 requests in all, split evenly over the ranks: strong scaling.  (--weak: 32 per rank.)
    B = SPEC["B"] if args.weak else max(1, SPEC["B"] // world)
    t_build = time.perf_counter()
    target, draft = build_spec_models(f"cuda:{local}")
    if args.quant:                       # weight-only quantised target (the INT8 / INT4 variants of the workload)
        target.quantize(args.quant)
    t_build = time.perf_counter() - t_build
    warm = max(args.warmup, 3)
    eng = _spec_engine(vn, target, draft, B, args, warm)
    prompts = spec_prompts(SPEC["B"] if args.weak else max(SPEC["B"], world), T0, SPEC["seed"], rank if args.weak else 0)
    prompts = prompts[:B] if args.weak else prompts[rank * B:(rank + 1) * B]
    ctx.sync()
    t_pre = time.perf_counter()
    eng.prefill(prompts)
    ctx.sync()
    t_pre = time.perf_counter() - t_pre
    for _ in range(warm):
        eng.step()
    # ---- timed region: K rounds, state resident on the device, no host synchronisation inside; repeated
    clocks = ClockSampler(local).start() if rank == 0 else None
    l0 = ctx.launch_count()
    reps, committed_rank = _time_engine(eng, ctx, dist, local, args.steps, warm)
    launches_per_repeat = (ctx.launch_count() - l0) // len(reps)
    clk = clocks.stop() if clocks else None
    ms = statistics.median(reps)
    committed = _sum_over_ranks(dist, committed_rank, local)
    value = committed / (ms * 1e-3)
    accept_rate = float(eng.accept_len.numpy().mean() / k)
    ctx_len = int(eng.t_cache.per_seq_lens.mean())
    launches = launches_per_repeat * args.steps // (args.steps + warm)

    # ---- end to end through the host-facing call: pinned host tokens in, committed tokens out, every round
    h_pair = ctx.pinned((B, 2), np.int64)
    h_len, h_tok = ctx.pinned((B,), np.int32), ctx.pinned((B, k + 1), np.int64)
    eng.rewind()
    for _ in range(warm):
        eng.step()
    eng.pair.copy_to_pinned_async(h_pair)
    ctx.sync()

    def e2e_step():
        eng.pair.copy_from_pinned_async(h_pair)     # the caller supplies the last committed tokens
        eng.step()
        eng.accept_len.copy_to_pinned_async(h_len)
        eng.out_tokens.copy_to_pinned_async(h_tok)
        eng.pair.copy_to_pinned_async(h_pair)
        ctx.sync()
        return int((h_tok >= 0).sum())

    e2e_step()
    n_e2e = args.steps
    barrier_sync(dist, ctx)
    t0 = time.perf_counter()
    got = 0
    for _ in range(n_e2e):
        got += e2e_step()
    barrier_sync(dist, ctx)
    e2e_s = max_over_ranks(dist, time.perf_counter() - t0, local)
    e2e = {"value": _sum_over_ranks(dist, got, local) / e2e_s, "unit": "tok/s", "steps": n_e2e,
           "h2d_bytes_per_step": int(h_pair.nbytes),
           "d2h_bytes_per_step": int(h_len.nbytes + h_tok.nbytes + h_pair.nbytes)}

    # ---- verify + sample part of a round: (a) timed as a replayed graph with CUDA events, (b) per-kernel
    # durations with CUDA events around every launch (eager; each pair of events adds a few microseconds,
    # so these give the SHARES, the graph timing gives the step time)
    n_prof = min(args.steps, 16)
    eng.rewind()
    for _ in range(warm):
        eng.step()
    lens0 = eng.t_cache.per_seq_lens.copy()
    eng.verify_accept_only(graph=False)
    eng.verify_accept_only(graph=True)
    v_reps = []
    for _ in range(5):
        eng.t_cache.set_lengths(lens0)                 # every repeat at the same context length
        eng._len_bound = int(lens0.max())
        v0, v1 = ctx.event(), ctx.event()
        v0.record()
        for _ in range(n_prof):
            eng.verify_accept_only(graph=True)
        v1.record()
        v_reps.append(v0.elapsed_ms(v1) / n_prof)
    eng.t_cache.set_lengths(lens0)
    eng._len_bound = int(lens0.max())
    step_ms = statistics.median(v_reps)
    ctx.profile(True)
    for _ in range(n_prof):
        eng.verify_accept_only()
    rep = ctx.profile_report()
    ctx.profile(False)
    prof_ms = max(sum(v["ms"] for v in rep.values()) / n_prof, 1e-9)
    gemm_ms = sum(v["ms"] for n, v in rep.items() if n.startswith("gemm_")) / n_prof * (step_ms / prof_ms)
    nbytes = spec_step_bytes(B, ctx_len)
    if args.quant:   # streamed weights: everything but the bf16 embedding table (the head has its own quantised copy)
        nbytes += target.param_bytes() - 248320 * 1024 * 2 - MATE_PARAMS * 2
    peak, peak_kind = peaks()
    achieved = nbytes / (step_ms * 1e-3) / 1e9
    top = sorted(rep.items(), key=lambda kv: -kv[1]["ms"])
    roofline = {"bound": "hbm", "kernel": "verify+sample step (all kernels of the target forward and acceptance)",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_kind": f"of {peak_kind}",
                "traffic": SPEC_STEP_TRAFFIC if (not args.quant and B == SPEC["B"]) else None,
                "step_ms": step_ms, "step_ms_repeats": v_reps, "algorithmic_bytes": nbytes,
                "gemm_ms": gemm_ms, "gemm_weight_gbs": MATE_PARAMS * 2 / (gemm_ms * 1e-3) / 1e9,
                "kernel_share": {n: v["ms"] / n_prof / prof_ms for n, v in top},
                "kernel_ms_per_step": {n: v["ms"] / n_prof for n, v in top},
                "kernel_launches_per_step": {n: v["launches"] / n_prof for n, v in top}}

    # ---- N > 1: the same models with 32 requests on every rank (weak scaling), and the sharded data path
    weak = sharded = None
    if world > 1 and not args.weak:
        if not args.no_weak:
            eng_w = _spec_engine(vn, target, draft, SPEC["B"], args, warm)
            eng_w.prefill(spec_prompts(SPEC["B"], T0, SPEC["seed"], rank))
            for _ in range(warm):
                eng_w.step()
            reps_w, c_w = _time_engine(eng_w, ctx, dist, local, args.steps, warm)
            ms_w = statistics.median(reps_w)
            weak = {"value": _sum_over_ranks(dist, c_w, local) / (ms_w * 1e-3), "unit": "tok/s",
                    "ms_per_step": ms_w / args.steps, "per_gpu_requests": SPEC["B"], "scaling": "weak",
                    **spread(reps_w, args.steps)}
            del eng_w
        if not args.no_sharded:
            sharded = _sharded_check(vn, target, draft, dist, ctx, local, world, rank)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        tps, secs, rounds = cpu_spec_sample()
        cpu = {"value": tps, "unit": "tok/s", "cores": blas_threads(), "kind": "port",
               "sample": f"1 of 32 requests, {rounds} rounds ({secs:.1f} s), full re-forward per round as the "
                         f"reference does; NumPy restatement (oracle/), fp32, {blas_threads()} BLAS threads"}
    sampler = None
    if rank == 0 and world == 1 and not args.no_sampler:
        del eng
        sampler = accept_quick(ctx)

    if rank == 0:
        print(json.dumps({
            "metric": "accepted tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak" if args.weak else "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": spec_config(args.quant),
            "timing": spread(reps, args.steps),
            "per_gpu_requests": B, "context_tokens": ctx_len,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clk,
            "accept_rate": accept_rate, "tokens_per_round_per_request": committed / world / B / args.steps,
            "prefill_s": t_pre, "weights_build_s": t_build, "sampler": sampler,
            "weak_32_per_gpu": weak, "sharded": sharded,
        }))
    if dist is not None:
        dist.destroy_process_group()


def spec_config(quant=None):
    """The `config` object of the default workload: the same in the device arm and in the CPU arm."""
    return {"workload": SPEC_WORKLOAD + (f", target weights {quant}" if quant else ""),
            "requests": SPEC["B"], "requests_split": "evenly over the ranks (32 / N per GPU)",
            "l2": "weights (2.2 GB) larger than L2, no flush", "step": "one speculative round over the batch"}


def run_sharded(args):
    """The vocabulary-sharded configuration: 32 requests per rank, 1024-token prompts, k = 6, T = 1.0, full-vocabulary
    rule, target linears INT8 (or --quant), LM head and acceptance split by vocabulary columns over the ranks: hidden
    rows, per-row statistics and picked tokens cross the ranks as NCCL all-gathers of device buffers on the library's
    stream, decisions stay on the device.  The same requests through the plain (unsharded) engine are timed beside it.
    Not the default benchmark line."""
    import versenext_b200 as vn
    from versenext_b200.comm import Comm
    from versenext_b200.sharded_engine import ShardedSpecEngine, rank_seed
    world, rank, local, dist = dist_setup(args.gpus)
    ctx = vn.Context.get(local)
    B, k, T0 = 32, 6, 1024
    scheme = args.quant or "int8"
    target, draft = build_spec_models(f"cuda:{local}")
    target.quantize(scheme)
    warm = max(args.warmup, 3)
    rounds = warm + args.steps + 8
    comm = Comm.from_torch_group(ctx) if dist is not None else None
    kw = dict(max_batch=B, max_seq=T0 + rounds * (k + 1) + 64, k=k, temperature=1.0, max_new_tokens=rounds * (k + 1))
    prompts = np.random.default_rng([5, rank]).integers(0, 248320, (B, T0)).astype(np.int64)
    eng = ShardedSpecEngine(target, draft, seed=5, comm=comm, **kw)
    eng.prefill(prompts)
    for _ in range(warm):
        eng.step()
    clocks = ClockSampler(local).start() if rank == 0 else None
    l0 = ctx.launch_count()
    reps, committed_rank = _time_engine(eng, ctx, dist, local, args.steps, warm)
    launches = (ctx.launch_count() - l0) // len(reps) * args.steps // (args.steps + warm)
    clk = clocks.stop() if clocks else None
    ms = statistics.median(reps)
    committed = _sum_over_ranks(dist, committed_rank, local)
    value = committed / (ms * 1e-3)
    ctx_len = int(eng.t_cache.per_seq_lens.mean())
    accept_rate = float(eng.accept_len.numpy().mean() / k)
    sharded_tokens = eng.history.numpy()[:, :args.steps].copy()
    del eng
    # the same requests, full head on every rank, same Philox numbers: the round the sharded one is measured against
    plain = vn.SpecEngine(target, draft, top_k=0, bonus=True, seed=rank_seed(5, rank), graph=True, **kw)
    plain.prefill(prompts)
    for _ in range(warm):
        plain.step()
    reps_p, _ = _time_engine(plain, ctx, dist, local, args.steps, warm)
    same = bool(np.array_equal(plain.history.numpy()[:, :args.steps], sharded_tokens))
    same_all = _sum_over_ranks(dist, 1.0 if same else 0.0, local) == world
    ms_p = statistics.median(reps_p)
    # streamed per round and rank: the quantised block weights, this rank's columns of the head, the K/V window
    head_bytes = 248320 * 1024 * (1 if scheme == "int8" else 0.5)
    nbytes = (target.param_bytes() - 248320 * 1024 * 2 - head_bytes * (1 - 1 / world)
              + 20 * B * min(ctx_len, 1024) * 2 * 512 * 2)
    peak, peak_kind = peaks()
    step_ms = ms / args.steps
    achieved = nbytes / (step_ms * 1e-3) / 1e9
    if rank == 0:
        print(json.dumps({
            "metric": "accepted tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"sharded: mate target with {scheme} linears + 2-layer D=256 draft, k=6, T=1.0, "
                                   f"full-vocabulary rule, 32 requests/GPU, 1024-token prompts, LM head and acceptance "
                                   f"split by vocabulary columns over the ranks (NCCL all-gathers of device buffers)",
                       "per_gpu_requests": B, "context_tokens": ctx_len, "step": "one speculative round",
                       "l2": "weights larger than L2, no flush"},
            "timing": spread(reps, args.steps),
            "unsharded_round": {"ms_per_step": ms_p / args.steps, "ratio_sharded_over_unsharded": ms / ms_p,
                                "same_tokens": bool(same_all), **spread(reps_p, args.steps)},
            "roofline": {"bound": "hbm", "kernel": "whole round (draft, verify, column-split head, sharded acceptance, "
                                                   "all-gathers)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "traffic": None, "algorithmic_bytes": nbytes},
            "cpu_baseline": None,
            # the sharded round keeps tokens, lengths and decisions on the device: there is no per-round host traffic
            # to time, so this workload carries no separate end-to-end figure
            "e2e": None,
            "gpu_launches": launches, "clocks": clk, "accept_rate": accept_rate,
            "tokens_per_round_per_request": committed / world / B / args.steps,
        }))
    if dist is not None:
        dist.destroy_process_group()


def accept_quick(ctx, steps=20):
    """sampler GB/s of the isolated acceptance op (second half of the headline metric)."""
    from versenext_b200 import sampling
    B, k, V = ACCEPT["B"], ACCEPT["k"], ACCEPT["V"]
    p, q, draft = make_accept_inputs(B, k, V, ACCEPT["seed"])
    pd, qd, dd = ctx.from_numpy(p), ctx.from_numpy(q), ctx.from_numpy(draft)
    out = (ctx.empty((B,), np.int32), ctx.empty((B, k + 1), np.int64))
    for i in range(3):
        sampling.accept(ctx, pd, qd, dd, seed=1234, offset=i, temperature=1.0, out=out)
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    for i in range(steps):
        sampling.accept(ctx, pd, qd, dd, seed=1234, offset=i, temperature=1.0, out=out)
    e1.record()
    ms = e0.elapsed_ms(e1) / steps
    peak, kind = peaks()
    gbs = accept_bytes(B, k, V) / (ms * 1e-3) / 1e9
    return {"metric": "sampler GB/s", "value": gbs, "unit": "GB/s", "ms_per_call": ms, "frac_of_hbm_peak": gbs / peak,
            "workload": "B=64 k=4 V=248320 fp32 logits, T=1.0"}


def run_reference_spec(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    budget = 150.0
    warm = max(args.warmup, 0)
    delta = args.workload == "delta"            # the delta-attention target: same round, other target model
    sampler = cpu_delta_sample if delta else cpu_spec_sample
    tps, secs, rounds = sampler(max_seconds=budget, rounds=max(1, args.steps), warmup=min(warm, 3))
    threads = blas_threads()
    sample = (f"1 of the 32 requests per step, {rounds} rounds run inside a {budget:.0f} s budget ({min(warm, 3)} untimed "
              f"warm-up rounds); full re-forward of [context, draft] per round as the reference does; NumPy restatement "
              f"of the reference algorithm (oracle/, kind 'port': the reference itself is Python and does not travel to "
              f"this machine), fp32, {threads} BLAS threads on {os.cpu_count()} host cores")
    print(json.dumps({
        "impl": "reference", "metric": "accepted tok/s", "value": tps, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": rounds, "warmup": warm, "ms_per_step": secs / max(rounds, 1) * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": ({"workload": DELTA_WORKLOAD, "requests": SPEC["B"], "step": "one speculative round over the batch"}
                   if delta else spec_config(args.quant)),
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------
# tree verification (16-node draft tree on a 2048-token cache, batch 8) and the small CPU-runnable configuration
# ---------------------------------------------------------------------------

TREE = dict(B=8, ctx=2048, parents=[-1, -1, -1, -1, 0, 0, 1, 1, 4, 4, 5, 5, 6, 6, 7, 7], seed=3)
TREE_WORKLOAD = ("tree: mate target (bf16), 16-node draft tree (4 roots, 2 children under each of the first two, 2 under "
                 "each of those), ancestor-bitmask attention on a 2048-token cache, batch 8")


def run_tree(args):
    import ctypes as C
    import versenext_b200 as vn
    from versenext_b200 import synthetic as S
    world, rank, local, dist = dist_setup(args.gpus)
    ctx = vn.Context.get(local)
    B, T0, parents = TREE["B"], TREE["ctx"], TREE["parents"]
    n = len(parents)
    tk = S.mate_kwargs()
    target = vn.VerseNexLM(dtype="bf16", device=f"cuda:{local}", **tk)
    S.load_random(target, tk, seed=0)
    if args.quant:
        target.quantize(args.quant)
    rng = np.random.default_rng([TREE["seed"], rank])
    cache = target.new_cache(B, T0 + n + 16)
    prompt = rng.integers(0, 248320, (B, T0)).astype(np.int64)
    for lo in range(0, T0, 512):
        target.forward_cached(prompt[:, lo:lo + 512], cache, want_logits=False, want_hidden=True, last_only=True)
        cache.commit(512, np.full(B, 512, np.int32))
    nodes = ctx.from_numpy(rng.integers(0, 248320, (B, n)).astype(np.int64))
    logits = ctx.empty((B, n, 248320), np.float32)
    pred = ctx.empty((B * n,), np.int64)

    def issue():
        target.forward_cached(nodes, cache, parents=parents, out_logits=logits)
        ctx._check(ctx.lib.vn_sample(ctx.handle, C.c_void_p(logits.ptr), 248320, B * n, 248320, 0.0, 0, None, 0, 0, 0, 0,
                                     C.c_void_p(pred.ptr)))

    issue()                                # eager once: buffers, attributes, the tree's masks
    ctx._check(ctx.lib.vn_graph_begin(ctx.handle))
    try:
        issue()
    finally:
        g = C.c_void_p()
        ctx._check(ctx.lib.vn_graph_end(ctx.handle, C.byref(g)))
    warm = max(args.warmup, 3)
    for _ in range(warm):
        ctx._check(ctx.lib.vn_graph_launch(ctx.handle, g))
    clocks = ClockSampler(local).start() if rank == 0 else None
    l0 = ctx.launch_count()
    issue()
    launches = (ctx.launch_count() - l0) * args.steps
    reps = timed_repeats(lambda: [ctx._check(ctx.lib.vn_graph_launch(ctx.handle, g)) for _ in range(args.steps)],
                         lambda: None, ctx, dist, local)
    clk = clocks.stop() if clocks else None
    ms = statistics.median(reps)
    step_ms = ms / args.steps
    target.check()
    nbytes = MATE_PARAMS * 2 + 20 * B * min(T0, 1024) * 2 * 512 * 2
    peak, peak_kind = peaks()
    achieved = nbytes / (step_ms * 1e-3) / 1e9
    # end to end: the tree's tokens from pinned host memory, the nodes' arg-max tokens back
    h_nodes, h_pred = ctx.pinned((B, n), np.int64), ctx.pinned((B * n,), np.int64)
    h_nodes[...] = nodes.numpy()

    def e2e_step():
        nodes.copy_from_pinned_async(h_nodes)
        ctx._check(ctx.lib.vn_graph_launch(ctx.handle, g))
        pred.copy_to_pinned_async(h_pred)
        ctx.sync()

    e2e_step()
    barrier_sync(dist, ctx)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier_sync(dist, ctx)
    e2e_s = max_over_ranks(dist, time.perf_counter() - t0, local)
    ctx._check(ctx.lib.vn_graph_destroy(ctx.handle, g))
    # the whole round with tree proposals: the 2-layer draft expands the tree, the target verifies it, the accepted
    # path is committed in both caches (TreeSpecEngine, greedy rule), replayed from a CUDA graph
    tree_engine = None
    if not args.quant:
        del cache, logits
        dk = S.draft_kwargs()
        draft = vn.VerseNexLM(dtype="bf16", device=f"cuda:{local}", **dk)
        S.load_random(draft, dk, seed=1)
        rounds = warm + args.steps + 4
        eng = vn.TreeSpecEngine(target, draft, parents, max_batch=B, max_seq=T0 + rounds * 4 + 64,
                                max_new_tokens=rounds * 4)
        eng.prefill(prompt)
        for _ in range(warm):
            eng.step()
        c0 = int(eng.counts().sum())
        e0, e1 = ctx.event(), ctx.event()
        e0.record()
        for _ in range(args.steps):
            eng.step()
        e1.record()
        barrier_sync(dist, ctx)
        t_ms = max_over_ranks(dist, e0.elapsed_ms(e1), local) / args.steps
        committed = int(eng.counts().sum()) - c0
        tree_engine = {"ms_per_round": t_ms, "tokens_per_round_per_request": committed / (args.steps * B),
                       "accepted_tok_s": committed * world / (t_ms * args.steps * 1e-3),
                       "what": "TreeSpecEngine round: draft tree expansion (3 levels) + target forward over 17 rows per "
                               "request + greedy path acceptance + cache commits, B = 8, context 2048"}
        # the same round with the stochastic walk (T = 0.8, top-k 50: top-k lists of all 136 target rows + rejection
        # sampling with fixed proposals)
        del eng
        eng = vn.TreeSpecEngine(target, draft, parents, max_batch=B, max_seq=T0 + rounds * 4 + 64,
                                max_new_tokens=rounds * 4, temperature=0.8, top_k=50, seed=3)
        eng.prefill(prompt)
        for _ in range(warm):
            eng.step()
        c0 = int(eng.counts().sum())
        e0, e1 = ctx.event(), ctx.event()
        e0.record()
        for _ in range(args.steps):
            eng.step()
        e1.record()
        barrier_sync(dist, ctx)
        t_ms = max_over_ranks(dist, e0.elapsed_ms(e1), local) / args.steps
        committed = int(eng.counts().sum()) - c0
        tree_engine["stochastic"] = {"ms_per_round": t_ms, "tokens_per_round_per_request": committed / (args.steps * B),
                                     "temperature": 0.8, "top_k": 50}
    if rank == 0:
        print(json.dumps({
            "metric": "verified tree nodes/s", "value": B * n * world * args.steps / (ms * 1e-3), "unit": "nodes/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": TREE_WORKLOAD + (f", target weights {args.quant}" if args.quant else ""),
                       "parents": parents, "step": "one target forward over the 16 nodes of every sequence + arg-max "
                       "per node", "l2": "weights (2.2 GB) larger than L2, no flush"},
            "timing": spread(reps, args.steps),
            "roofline": {"bound": "hbm", "kernel": "tree verify step (all kernels of the target forward over 128 node "
                         "rows, LM head, arg-max)", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": None, "step_ms": step_ms,
                         "algorithmic_bytes": nbytes, "target_ms": 0.53},
            "cpu_baseline": None,
            "e2e": {"value": B * n * world * args.steps / e2e_s, "unit": "nodes/s",
                    "h2d_bytes_per_step": int(h_nodes.nbytes), "d2h_bytes_per_step": int(h_pred.nbytes)},
            "gpu_launches": launches, "clocks": clk, "tree_engine": tree_engine,
        }))
    if dist is not None:
        dist.destroy_process_group()


SMALL = dict(vocab_size=256, dim=64, n_layer=2, n_head=4, n_kv_head=2, window_size=32, num_global_tokens=4,
             use_alibi=True, use_rope=False, max_seq_len=256, tie_weights=True)
SMALL_WORKLOAD = ("small: VerseNexLM dim 64, 2 TriSparse layers, vocab 256, fp32 + 1-layer draft, k=4, greedy, batch 1, "
                  "32-token prompt, 128 generated tokens")


def _small_weights():
    from versenext_b200 import synthetic as S
    tk, dk = dict(SMALL), dict(SMALL, n_layer=1)
    t_sd = dict(S.random_tensors(tk, seed=0, init_std=0.2))
    d_sd = dict(S.random_tensors(dk, seed=1, init_std=0.2))
    d_sd["tok_emb.weight"] = t_sd["tok_emb.weight"]
    return tk, dk, t_sd, d_sd


def cpu_small_run():
    """The whole small configuration on the host (NumPy restatement of the reference loop): tok/s, seconds."""
    from oracle import model as OM
    from oracle import spec as OS
    tk, dk, t_sd, d_sd = _small_weights()
    t_cfg, d_cfg = OM.Config(**tk), OM.Config(**dk)
    t_sd["head.weight"], d_sd["head.weight"] = t_sd["tok_emb.weight"], d_sd["tok_emb.weight"]
    prompt = np.random.default_rng(0).integers(0, 256, (1, 32)).astype(np.int64)
    t0 = time.perf_counter()
    st = OS.generate(t_sd, t_cfg, d_sd, d_cfg, prompt, 4, 128, temperature=0.0, bonus=False)
    dt = time.perf_counter() - t0
    return 128 / dt, dt, st


DELTA_WORKLOAD = ("delta: the shipped mate preset with delta attention (D=1024, L=32: 4 vda + 26 gmla + 2 dsa, all SwiGLU, "
                  "16 heads / 8 KV heads, window 1024, 128 sinks, anchor 128, V=248320, bf16) + 2-layer D=256 draft, "
                  "k=4, T=0.8, top-k 50, 32 requests of 512-token prompts")


def delta_kwargs():
    """Constructor arguments of the shipped mate preset (spark/mate/config/cometspark_mate.yml: use_vda, 32 layers,
    layer kinds from build_verse_delta_pattern)."""
    import versenext_b200 as vn
    from versenext_b200 import synthetic as S
    return S.mate_kwargs(n_layer=32, layer_pattern=vn.build_verse_delta_pattern(32), anchor_interval=128)


def cpu_delta_sample(max_seconds=25.0, rounds=2, warmup=1):
    """The delta workload on the host (NumPy restatement): one request, full re-forward every round."""
    from oracle import model as OM
    from oracle import spec as OS
    from versenext_b200 import synthetic as S
    tk, dk = delta_kwargs(), S.draft_kwargs()
    t_cfg = OM.Config(**tk)
    d_cfg = OM.Config(**dk)
    t_sd = dict(S.random_tensors(tk, seed=0))
    t_sd["head.weight"] = t_sd["tok_emb.weight"]
    d_sd = dict(S.random_tensors(dk, seed=1))
    d_sd["head.weight"] = d_sd["tok_emb.weight"]
    seq = spec_prompts(1, SPEC["prompt"], SPEC["seed"])
    t0, done, committed = None, 0, 0
    for i in range(warmup + rounds):
        if i == warmup:
            t0 = time.perf_counter()
        if t0 is not None and time.perf_counter() - t0 > max_seconds:
            break
        st = OS.generate(t_sd, t_cfg, d_sd, d_cfg, seq, SPEC["k"], 10 ** 6, temperature=SPEC["temperature"],
                         top_k=SPEC["top_k"], seed=SPEC["seed"], bonus=True, max_rounds=1)
        new_seq = st["tokens"][0]
        if i >= warmup:
            committed += new_seq.shape[1] - seq.shape[1]
            done += 1
        seq = new_seq
    dt = time.perf_counter() - t0
    return committed / dt, dt, done


def run_delta(args):
    """The speculative round with a target made of delta attention layers (one GPU, or replicas)."""
    import versenext_b200 as vn
    from versenext_b200 import synthetic as S
    world, rank, local, dist = dist_setup(args.gpus)
    ctx = vn.Context.get(local)
    k, T0, B = SPEC["k"], SPEC["prompt"], SPEC["B"]
    tk, dk = delta_kwargs(), S.draft_kwargs()
    target = vn.VerseNexLM(dtype="bf16", device=f"cuda:{local}", **tk)
    S.load_random(target, tk, seed=0)
    if args.quant:                       # the shipped preset's weight-only INT4 (or INT8) on the same layers
        target.quantize(args.quant)
    draft = vn.VerseNexLM(dtype="bf16", device=f"cuda:{local}", **dk)
    S.load_random(draft, dk, seed=1)
    warm = max(args.warmup, 3)
    eng = _spec_engine(vn, target, draft, B, args, warm)
    ctx.sync()
    t_pre = time.perf_counter()
    eng.prefill(spec_prompts(B, T0, SPEC["seed"], rank))
    ctx.sync()
    t_pre = time.perf_counter() - t_pre
    for _ in range(warm):
        eng.step()
    clocks = ClockSampler(local).start() if rank == 0 else None
    l0 = ctx.launch_count()
    reps, committed_rank = _time_engine(eng, ctx, dist, local, args.steps, warm)
    launches = (ctx.launch_count() - l0) // len(reps) * args.steps // (args.steps + warm)
    clk = clocks.stop() if clocks else None
    ms = statistics.median(reps)
    value = _sum_over_ranks(dist, committed_rank, local) / (ms * 1e-3)
    ctx_len = int(eng.t_cache.per_seq_lens.mean())
    # verify + sample step as a replayed graph, then per-kernel shares with events around every launch
    n_prof = min(args.steps, 16)
    eng.rewind()
    for _ in range(warm):
        eng.step()
    lens0 = eng.t_cache.per_seq_lens.copy()
    eng.verify_accept_only(graph=False)
    eng.verify_accept_only(graph=True)
    v_reps = []
    for _ in range(5):
        eng.t_cache.set_lengths(lens0)
        eng._len_bound = int(lens0.max())
        v0, v1 = ctx.event(), ctx.event()
        v0.record()
        for _ in range(n_prof):
            eng.verify_accept_only(graph=True)
        v1.record()
        v_reps.append(v0.elapsed_ms(v1) / n_prof)
    eng.t_cache.set_lengths(lens0)
    eng._len_bound = int(lens0.max())
    step_ms = statistics.median(v_reps)
    ctx.profile(True)
    for _ in range(n_prof):
        eng.verify_accept_only()
    rep = ctx.profile_report()
    ctx.profile(False)
    prof_ms = max(sum(v["ms"] for v in rep.values()) / n_prof, 1e-9)
    # algorithmic bytes: every target weight once + the K / V every module has to read (a module of a context of at
    # most 1024 keys reads all of it; 40 modules: 3 per vda layer, 1 per gmla / dsa layer; 2 x 512 values per key)
    params = S.param_count(tk)
    n_mod = sum(3 if kind == "vda" else 1 for kind in tk["layer_pattern"])
    nbytes = params * 2 + n_mod * B * min(ctx_len, 1024) * 2 * 512 * 2
    if args.quant:                       # streamed weights: what the quantised model holds, minus the embedding table
        nbytes += target.param_bytes() - 248320 * 1024 * 2 - params * 2
    peak, peak_kind = peaks()
    achieved = nbytes / (step_ms * 1e-3) / 1e9
    top = sorted(rep.items(), key=lambda kv: -kv[1]["ms"])
    roofline = {"bound": "hbm", "kernel": "verify+sample step (all kernels of the target forward and acceptance)",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                "traffic": None, "step_ms": step_ms, "step_ms_repeats": v_reps, "algorithmic_bytes": nbytes,
                "kernel_share": {n: v["ms"] / n_prof / prof_ms for n, v in top},
                "kernel_ms_per_step": {n: v["ms"] / n_prof for n, v in top},
                "kernel_launches_per_step": {n: v["launches"] / n_prof for n, v in top}}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        tps, secs, rounds = cpu_delta_sample()
        cpu = {"value": tps, "unit": "tok/s", "cores": blas_threads(), "kind": "port",
               "sample": f"1 of 32 requests, {rounds} rounds ({secs:.1f} s), full re-forward per round as the "
                         f"reference does; NumPy restatement (oracle/), fp32, {blas_threads()} BLAS threads"}
    if rank == 0:
        print(json.dumps({
            "metric": "accepted tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": DELTA_WORKLOAD + (f", target weights {args.quant}" if args.quant else ""), "requests": B,
                       "l2": "weights and K / V read per step (2.7 GB dense) larger than L2, no flush",
                       "step": "one speculative round over the batch"},
            "timing": spread(reps, args.steps), "context_tokens": ctx_len, "target_params": params,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": None, "gpu_launches": launches, "clocks": clk,
            "accept_rate": float(eng.accept_len.numpy().mean() / k), "prefill_s": t_pre,
        }))
    if dist is not None:
        dist.destroy_process_group()


def run_layer(args):
    """One MoD + one TriSparse layer of the mate shapes (D=1024, 16 heads / 8 KV heads, window 1024, 128 sinks) with a
    small vocabulary: the per-layer kernels of the verify step on a case small enough for a full ncu capture
    (about 60 MB of weights, 0.3 GB of KV cache).  32 sequences at context 1100, 5 new rows each, as in the round."""
    import versenext_b200 as vn
    from versenext_b200 import synthetic as S
    world, rank, local, dist = dist_setup(args.gpus)
    ctx = vn.Context.get(local)
    pattern = args.pattern.split(",")          # default: one MoD + one TriSparse layer; e.g. --pattern vda,gmla
    kw = S.mate_kwargs(vocab_size=8192, n_layer=len(pattern), layer_pattern=pattern, max_seq_len=2048)
    m = vn.VerseNexLM(dtype="bf16", device=f"cuda:{local}", **kw)
    S.load_random(m, kw, seed=3)
    B, T0, Tn = 32, args.context, 5
    rng = np.random.default_rng(5)
    cache = m.new_cache(B, T0 + 64)
    for lo in range(0, T0, 220):                       # prefill in pieces of 220 positions
        m.forward_cached(rng.integers(0, 8192, (B, 220)).astype(np.int64), cache, want_logits=False)
        cache.commit(220, np.full(B, 220, np.int32))
    nxt = ctx.from_numpy(rng.integers(0, 8192, (B, Tn)).astype(np.int64))
    out = ctx.empty((B, Tn, 8192), np.float32)
    for _ in range(max(args.warmup, 3)):
        m.forward_cached(nxt, cache, out_logits=out)
    barrier_sync(dist, ctx)
    l0 = ctx.launch_count()
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    for _ in range(args.steps):
        m.forward_cached(nxt, cache, out_logits=out)
    e1.record()
    barrier_sync(dist, ctx)
    ms = max_over_ranks(dist, e0.elapsed_ms(e1), local) / args.steps
    if rank == 0:
        print(json.dumps({"metric": "two-layer slice forward", "value": ms, "unit": "ms", "n_gpus": world,
                          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
                          "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": f"layer: layers {args.pattern} of the mate shapes, V=8192, "
                                                 f"32 sequences at context {T0}, 5 new rows each (eager launches)"},
                          "gpu_launches": ctx.launch_count() - l0}))
    if dist is not None:
        dist.destroy_process_group()


def run_small(args):
    import versenext_b200 as vn
    world, rank, local, dist = dist_setup(args.gpus)
    ctx = vn.Context.get(local)
    tk, dk, t_sd, d_sd = _small_weights()
    target = vn.VerseNexLM(dtype="f32", device=f"cuda:{local}", **tk)
    target.load_state_dict(t_sd)
    draft = vn.VerseNexLM(dtype="f32", device=f"cuda:{local}", **dk)
    draft.load_state_dict(d_sd)
    prompt = np.random.default_rng(0).integers(0, 256, (1, 32)).astype(np.int64)
    eng = vn.SpecEngine(target, draft, max_batch=1, max_seq=256, k=4, temperature=0.0, bonus=False, max_new_tokens=160)
    toks, st = eng.generate(prompt, 128)
    warm = max(args.warmup, 3)
    for _ in range(warm):
        eng.generate(prompt, 128)
    clocks = ClockSampler(local).start() if rank == 0 else None
    barrier_sync(dist, ctx)
    l0 = ctx.launch_count()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        toks, st = eng.generate(prompt, 128)          # prompt from the host, tokens back to the host: end to end
    barrier_sync(dist, ctx)
    secs = max_over_ranks(dist, time.perf_counter() - t0, local)
    launches = ctx.launch_count() - l0
    clk = clocks.stop() if clocks else None
    # device-resident part: the rounds alone, after prefill
    eng.prefill(prompt)
    for _ in range(3):
        eng.step()
    reps = timed_repeats(lambda: [eng.step() for _ in range(32)], lambda: (eng.rewind(), eng.step()), ctx, dist, local,
                         min_total_ms=200.0)
    round_ms = statistics.median(reps) / 32
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        tps, dt, cst = cpu_small_run()
        cpu = {"value": tps, "unit": "tok/s", "cores": blas_threads(), "kind": "port",
               "sample": f"the whole configuration: 128 tokens in {cst['rounds']} rounds ({dt:.1f} s), full re-forward per "
                         "round as the reference does; NumPy restatement (oracle/)",
               "same_tokens_as_device": bool(np.array_equal(cst["tokens"], toks))}
    if rank == 0:
        value = 128 * world * args.steps / secs
        print(json.dumps({
            "metric": "accepted tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": SMALL_WORKLOAD, "step": "one whole generation of 128 tokens (prefill + rounds)",
                       "l2": "model fits in L2: latency-bound by construction"},
            "roofline": None, "round_ms": round_ms, "rounds": st["rounds"], "cpu_baseline": cpu,
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": int(prompt.nbytes),
                    "d2h_bytes_per_step": int(toks.nbytes)},
            "gpu_launches": launches, "clocks": clk,
        }))
    if dist is not None:
        dist.destroy_process_group()


def run_reference_small(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    tps, dt, st = cpu_small_run()
    sample = f"the whole configuration once ({dt:.1f} s, {st['rounds']} rounds), NumPy restatement (oracle/), {blas_threads()} BLAS threads"
    print(json.dumps({
        "impl": "reference", "metric": "accepted tok/s", "value": tps, "unit": "tok/s", "n_gpus": args.gpus, "steps": 1,
        "warmup": 0, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": SMALL_WORKLOAD, "step": "one whole generation of 128 tokens (prefill + rounds)",
                   "l2": "model fits in L2: latency-bound by construction"},
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": blas_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_reference(args):
    world, rank, local, _ = 1, int(os.environ.get("RANK", "0")), 0, None
    if rank != 0:
        return
    n_seq = 8
    k, V = ACCEPT["k"], ACCEPT["V"]
    from oracle import accept as OA
    from oracle import philox as OP
    p, q, draft = make_accept_inputs(n_seq, k, V, ACCEPT["seed"])
    ua, us = OP.uniforms_for_call(ACCEPT["seed"], 0, n_seq, k)
    for _ in range(max(args.warmup, 0)):
        OA.accept(p[:1], q[:1], draft[:1], ua[:1], us[:1], 1.0, 0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        OA.accept(p, q, draft, ua, us, ACCEPT["temperature"], 0)
    dt = time.perf_counter() - t0
    gbs = accept_bytes(n_seq, k, V) * args.steps / dt / 1e9
    sample = f"{n_seq} of 64 sequences per step (k=4, V=248320), NumPy restatement of the reference algorithm"
    print(json.dumps({
        "impl": "reference", "metric": "sampler GB/s", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "accept: B=64 k=4 V=248320 fp32 logits, T=1.0, Philox seed 1234",
                   "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------
# B200 arm
# ---------------------------------------------------------------------------

def run_accept(args):
    import versenext_b200 as vn
    from versenext_b200 import sampling
    world, rank, local, dist = dist_setup(args.gpus)
    ctx = vn.Context.get(local)
    B, k, V = ACCEPT["B"], ACCEPT["k"], ACCEPT["V"]
    p, q, draft = make_accept_inputs(B, k, V, ACCEPT["seed"] + rank)
    pd, qd, dd = ctx.from_numpy(p), ctx.from_numpy(q), ctx.from_numpy(draft)
    out = (ctx.empty((B,), np.int32), ctx.empty((B, k + 1), np.int64))
    nbytes = accept_bytes(B, k, V)

    def step(i):
        sampling.accept(ctx, pd, qd, dd, seed=ACCEPT["seed"], offset=i, temperature=ACCEPT["temperature"],
                        bonus=True, out=out)

    for i in range(max(args.warmup, 3)):
        step(i)
    # ---- device-resident timed region (inputs 572 MB > 126 MB L2: no flush needed)
    clocks = ClockSampler(local).start() if rank == 0 else None
    barrier_sync(dist, ctx)
    l0 = ctx.launch_count()
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    ms = e0.elapsed_ms(e1)
    barrier_sync(dist, ctx)
    launches = ctx.launch_count() - l0
    clk = clocks.stop() if clocks else None
    ms = max_over_ranks(dist, ms, local)
    value = nbytes * world * args.steps / (ms * 1e-3) / 1e9

    # ---- per-kernel durations (CUDA events around each launch), separate pass
    ctx.profile(True)
    for i in range(args.steps):
        step(i)
    rep = ctx.profile_report()
    ctx.profile(False)
    dom = next(n for n in rep if "accept_stats_kernel" in n)
    dom_ms = rep[dom]["ms"] / rep[dom]["launches"]
    peak, peak_kind = peaks()
    achieved = nbytes / (dom_ms * 1e-3) / 1e9
    total_k = sum(v["ms"] for v in rep.values())
    roofline = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                "kernel_ms": dom_ms, "algorithmic_bytes": nbytes,
                "kernel_shares": {n: v["ms"] / total_k for n, v in rep.items()}}
    # DRAM bytes of one launch of the dominant kernel, from the ncu capture summarised in
    # profiles/accept_stats_kernel_ncu_full.txt (dram__bytes_read.sum + dram__bytes_write.sum); it scales with
    # the rows processed, so it is only quoted for the configuration that was captured
    if (B, k, V) == (64, 4, 248320):
        roofline["traffic"] = 572177920 + 4024064
        roofline["traffic_source"] = "profiles/accept_stats_kernel_ncu_full.txt"

    # ---- end to end: pinned host logits -> device -> op -> host result, every step
    hp, hq, hd = ctx.pinned(p.shape, np.float32), ctx.pinned(q.shape, np.float32), ctx.pinned(draft.shape, np.int64)
    hp[...] = p
    hq[...] = q
    hd[...] = draft
    h_len, h_tok = ctx.pinned((B,), np.int32), ctx.pinned((B, k + 1), np.int64)

    def e2e_step(i):
        pd.copy_from_pinned_async(hp)
        qd.copy_from_pinned_async(hq)
        dd.copy_from_pinned_async(hd)
        step(i)
        out[0].copy_to_pinned_async(h_len)
        out[1].copy_to_pinned_async(h_tok)
        ctx.sync()

    e2e_step(0)
    n_e2e = max(2, min(args.steps, 5))
    barrier_sync(dist, ctx)
    t0 = time.perf_counter()
    for i in range(n_e2e):
        e2e_step(i)
    barrier_sync(dist, ctx)
    e2e_s = max_over_ranks(dist, time.perf_counter() - t0, local)
    e2e = {"value": nbytes * world * n_e2e / e2e_s / 1e9, "unit": "GB/s", "steps": n_e2e,
           "h2d_bytes_per_step": int(hp.nbytes + hq.nbytes + hd.nbytes),
           "d2h_bytes_per_step": int(h_len.nbytes + h_tok.nbytes)}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        gbs, secs = cpu_accept_sample(8)
        cpu = {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "port",
               "sample": f"8 of 64 sequences, one call ({secs:.2f} s), NumPy restatement (oracle/accept.py)"}

    if rank == 0:
        print(json.dumps({
            "metric": "sampler GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "accept: B=64 k=4 V=248320 fp32 logits, T=1.0, Philox seed 1234",
                       "per_gpu_batch": B, "l2": "inputs (572 MB) larger than L2, no flush"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clk,
            "accept_rate": float(out[0].numpy().mean() / k),
        }))
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="spec", choices=["spec", "accept", "sharded", "tree", "small", "layer", "delta"])
    ap.add_argument("--weak", action="store_true",
                    help="spec workload: 32 requests on every rank (default: the configuration's 32 split over the ranks)")
    ap.add_argument("--no-weak", action="store_true", help="N > 1: skip the extra 32-per-GPU measurement")
    ap.add_argument("--no-sharded", action="store_true", help="N > 1: skip the sharded-head check")
    ap.add_argument("--quant", default=None, choices=["int8", "int4", "int4g128"],
                    help="spec workload: quantise the target's linear weights (not the default benchmark line)")
    ap.add_argument("--pattern", default="mod,trisparse", help="layer workload: comma-separated layer kinds")
    ap.add_argument("--context", type=int, default=1100, help="layer workload: cached positions (a multiple of 220)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-sampler", action="store_true", help="spec workload: skip the sampler GB/s measurement")
    args = ap.parse_args()
    if args.impl == "reference":
        {"accept": run_reference, "small": run_reference_small}.get(args.workload, run_reference_spec)(args)
    else:
        {"spec": run_spec, "accept": run_accept, "sharded": run_sharded, "tree": run_tree,
         "small": run_small, "layer": run_layer, "delta": run_delta}[args.workload](args)


if __name__ == "__main__":
    main()
