#!/usr/bin/env python
"""Benchmark of the speculative-decoding hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload accept]

Prints ONE JSON line (rank 0).  Workloads:

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

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ACCEPT = dict(B=64, k=4, V=248320, seed=1234, temperature=1.0)


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


def dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
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
    dom = "accept_stats_kernel<true>"
    dom_ms = rep[dom]["ms"] / rep[dom]["launches"]
    peak, peak_kind = peaks()
    achieved = nbytes / (dom_ms * 1e-3) / 1e9
    total_k = sum(v["ms"] for v in rep.values())
    roofline = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                "kernel_ms": dom_ms, "algorithmic_bytes": nbytes,
                "kernel_shares": {n: v["ms"] / total_k for n, v in rep.items()}}
    tpath = os.path.join(ROOT, "profiles", "accept_traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            roofline["traffic"] = json.load(f).get("dram_bytes_per_launch")

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
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="accept", choices=["accept"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_accept(args)


if __name__ == "__main__":
    main()
