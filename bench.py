#!/usr/bin/env python
"""Benchmark of the attention-with-scores hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-ops]

Workload (config.workload = "cfg2"): fused attention_with_scores, fp16, B=1,
Hq=Hkv=32, S=1024, D=128, causal, fp32 scores (1,32,1024,1024) -- the
configuration the headline metric is quoted on.  One step = one call of the
public operator on one batch of synthetic N(0,1) inputs.  With N > 1 ranks
(torchrun, one process per GPU) every rank runs the same per-GPU workload on
its own (batch x kv-head) units: weak scaling, no data-path collective.

The JSON line carries the score-write rate (`value`, GB/s), the roofline of the
dominant kernel, the same metric end to end from pinned host buffers (`e2e`),
the CPU oracle timed on this host (`cpu_baseline`), sampled clocks, and a table
of the other operators on their configurations (`ops`).

`--impl reference` times the reference's own CPU path for this operator (the
naive PyTorch attention, restated in oracle/oracle.py) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG2 = dict(B=1, Hq=32, Hk=32, S=1024, D=128, dtype=torch.float16, causal=True)
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel on this
# workload, from the committed ncu summary of that kernel on this workload (None = not captured)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 112_927_744  # 25.48 MB read + 87.45 MB written (the rest stays dirty in L2)
N_SETS = 4  # rotating buffer sets: 4 x (134 MB scores + 8 MB out + 25 MB inputs) > 126 MB of L2


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm=float(d["hbm_gbs"]), tensor=float(d["bf16_tflops"]),
                    tensor_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), src="measured")
    return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, src="fallback")


def algorithmic(cfg, op="scores", split=None):
    """FLOPs and bytes of one call: 4*pairs*D per (b, q head) (+2*extra pairs for a second q.k^T);
    bytes = q, out, k, v once + the operator's fp32 outputs."""
    B, Hq, Hk, S, D = cfg["B"], cfg["Hq"], cfg["Hk"], cfg["S"], cfg["D"]
    pairs = S * (S + 1) // 2 if cfg["causal"] else S * S
    extra = 0
    out_bytes = 0
    if op == "scores":
        out_bytes = B * Hq * S * S * 4
    elif op in ("row_sum",):
        out_bytes = B * Hq * S * 4
    elif op in ("col_sum", "col_sum_sequential"):
        out_bytes = B * Hk * S * 4
    elif op == "softmax_col_sum":
        extra = pairs
        out_bytes = B * Hk * S * 4
    elif op == "cross_qk":
        out_bytes = B * Hk * split * 4
    elif op == "cross_softmax":
        extra = (S - split) * split
        out_bytes = B * Hk * split * 4
    elif op == "cross_softmax_buffered":
        out_bytes = B * Hk * split * 4 + 2 * 4 * B * Hq * (S - split) * split
    flops = B * Hq * D * (4 * pairs + 2 * extra)
    io = 2 * B * Hq * S * D * 2 + 2 * B * Hk * S * D * 2
    return flops, io + out_bytes


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index), "-f", self.path], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.split(",") for r in open(self.path).read().strip().splitlines() if r.strip()]
            os.unlink(self.path)
        except Exception:
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def make_inputs(cfg, seed, device, S=None):
    S = cfg["S"] if S is None else S
    if device is not None and cfg["B"] * cfg["Hq"] * S * cfg["D"] > (1 << 27):
        # very large configs (cfg5): draw on the device, the CPU generator would take many seconds
        g = torch.Generator(device=device).manual_seed(seed)
        mk = lambda h: torch.randn(cfg["B"], h, S, cfg["D"], device=device, generator=g)  # noqa: E731
        q, k, v = mk(cfg["Hq"]), mk(cfg["Hk"]), mk(cfg["Hk"])
        if cfg.get("vdist") == "uniform":
            v = torch.rand(cfg["B"], cfg["Hk"], S, cfg["D"], device=device, generator=g) * 2 - 1
        return q.to(cfg["dtype"]), k.to(cfg["dtype"]), v.to(cfg["dtype"])
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(cfg["B"], cfg["Hq"], S, cfg["D"], generator=g).to(cfg["dtype"])
    k = torch.randn(cfg["B"], cfg["Hk"], S, cfg["D"], generator=g).to(cfg["dtype"])
    v = torch.randn(cfg["B"], cfg["Hk"], S, cfg["D"], generator=g).to(cfg["dtype"])
    if cfg.get("vdist") == "uniform":
        v = (torch.rand(cfg["B"], cfg["Hk"], S, cfg["D"], generator=g) * 2 - 1).to(cfg["dtype"])
    elif cfg.get("vscale"):
        v = (v.float() * cfg["vscale"]).to(cfg["dtype"])
    if device is None:
        return q, k, v
    return q.to(device), k.to(device), v.to(device)


def cpu_reference_time(cfg, runs):
    """The reference's naive CPU path (oracle port) on the host cores: median seconds per call."""
    from oracle import oracle as orc
    q, k, v = make_inputs(cfg, 0, None)
    q, k, v = q.float(), k.float(), v.float()
    orc.naive_attention_with_scores(q, k, v, cfg["causal"])  # warm-up
    ts = []
    for _ in range(runs):
        t0 = time.perf_counter()
        orc.naive_attention_with_scores(q, k, v, cfg["causal"])
        ts.append(time.perf_counter() - t0)
    return ts


def check_parity(buffers, cfg):
    """out / scores of one buffer set against the CPU oracle (the checker, outside every timed region)."""
    from oracle import oracle as orc
    q, k, v, out, scores = buffers
    torch.cuda.synchronize()
    ref_out, ref_scores = orc.naive_attention_with_scores(q.cpu(), k.cpu(), v.cpu(), cfg["causal"])
    ok_out, out_err = orc.check_out(out.cpu(), ref_out)
    ok_sc, viol, ok_mask = orc.check_scores(scores.cpu(), ref_scores)
    return {"checked": True, "ok": bool(ok_out and ok_sc and ok_mask), "out_max_abs": out_err, "out_tol": orc.OUT_ATOL,
            "scores_max_viol": viol, "scores_tol": "1e-3*|ref| + 1e-4 (violation <= 0 passes)",
            "mask_bit_exact": bool(ok_mask), "against": "oracle/oracle.py naive_attention_with_scores, whole tensors"}


def run_reference(args, rank, emit):
    if rank != 0:
        return
    # all the host threads this process may use (torchrun exports OMP_NUM_THREADS=1 for its workers)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    cfg = CFG2
    flops, nbytes = algorithmic(cfg)
    score_bytes = cfg["B"] * cfg["Hq"] * cfg["S"] * cfg["S"] * 4
    ts = cpu_reference_time(cfg, max(1, args.warmup))  # warm-up calls
    t0 = time.perf_counter()
    ts = cpu_reference_time(cfg, args.steps)
    total = sum(ts)
    sec = total / args.steps
    val = score_bytes / sec / 1e9
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "attention_with_scores score-write rate", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg2", "op": "attention_with_scores", "B": 1, "Hq": 32, "Hk": 32, "S": 1024,
                   "D": 128, "causal": True},
        "tflops": flops / sec / 1e12,
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"whole cfg2 problem, {args.steps} calls of the naive PyTorch path "
                                   f"(oracle port) on {cores} threads of {os.cpu_count()} logical CPUs"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def time_op(fn, iters, warmup):
    """Mean CUDA-event time of one call: one event pair around `iters` calls queued back to back behind a
    spin kernel, so that neither host enqueue latency nor per-call event records are inside the pair."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(int(2e6))
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def ops_table(F, device, pk):
    """The other operators on their benchmark configurations (mean ms of 30 back-to-back calls each)."""
    rows = []
    cfg3 = dict(B=1, Hq=28, Hk=4, S=4096, D=128, dtype=torch.bfloat16, causal=True, vscale=0.5)
    cfg4 = dict(B=2, Hq=32, Hk=8, S=4096, D=128, dtype=torch.float16, causal=True)
    cfg5 = dict(B=4, Hq=32, Hk=8, S=16384, D=128, dtype=torch.bfloat16, causal=False, vdist="uniform")
    plans = [
        ("cfg3", cfg3, None, [("attention", F.attention), ("row_sum", F.attention_with_row_sum),
                              ("col_sum", F.attention_with_col_sum),
                              ("col_sum_sequential", F.attention_with_col_sum_sequential),
                              ("softmax_col_sum", F.attention_with_softmax_col_sum)]),
        ("cfg4", cfg4, 3072, [("cross_qk", F.attention_cross_token_qk_sum),
                              ("cross_softmax", F.attention_cross_token_softmax_sum),
                              ("cross_softmax_buffered", F.attention_cross_token_softmax_sum_buffered)]),
        ("cfg5", cfg5, None, [("attention", F.attention), ("softmax_col_sum", F.attention_with_softmax_col_sum)]),
        ("cfg5", cfg5, 12288, [("cross_softmax", F.attention_cross_token_softmax_sum)]),
    ]
    for name, cfg, split, ops in plans:
        q, k, v = make_inputs(cfg, 0, device)
        for op, fn in ops:
            if split is None:
                call = lambda: fn(q, k, v, cfg["causal"])  # noqa: E731
            else:
                call = lambda: fn(q, k, v, split, cfg["causal"])  # noqa: E731
            ms = time_op(call, 30, 3)
            flops, nbytes = algorithmic(cfg, "scores" if op == "attention" else op, split)
            if op == "attention":
                nbytes -= cfg["B"] * cfg["Hq"] * cfg["S"] * cfg["S"] * 4
            t_tensor = flops / (pk["tensor"] * 1e12)
            t_hbm = nbytes / (pk["hbm"] * 1e9)
            bound = "tensor" if t_tensor >= t_hbm else "hbm"
            row = {"config": name, "op": op, "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                   "gbs": nbytes / (ms * 1e-3) / 1e9, "bound": bound,
                   "frac": max(t_tensor, t_hbm) / (ms * 1e-3), "backend": F.last_backend()}
            if bound == "tensor" and ms >= 2.0:
                # 30 calls of milliseconds each run under the power cap like the seconds-long matmul loop behind
                # the sustained peak: that is the denominator for this row; `frac` (burst peak) is kept beside it
                row["frac_of_sustained_peak"] = flops / (ms * 1e-3) / 1e12 / pk["tensor_sustained"]
                row["peak_that_applies"] = "sustained (%.0f TFLOP/s); frac is against the burst peak" % pk["tensor_sustained"]
            rows.append(row)
        del q, k, v
    rows += extra_rows(F, device, pk)
    return rows


def extra_rows(F, device, pk):
    """Backward pass, score-only operator and split-KV decoding, same timing as the rows above."""
    rows = []

    def add(config, op, ms, flops, nbytes, note=None):
        t_tensor, t_hbm = flops / (pk["tensor"] * 1e12), nbytes / (pk["hbm"] * 1e9)
        r = {"config": config, "op": op, "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "gbs": nbytes / (ms * 1e-3) / 1e9,
             "bound": "tensor" if t_tensor >= t_hbm else "hbm", "frac": max(t_tensor, t_hbm) / (ms * 1e-3),
             "backend": F.last_backend()}
        if note:
            r["note"] = note
        rows.append(r)

    # backward of attention on cfg3: dq, dk, dv from (q, k, v, out, L, dout); 5 GEMMs per (query, key) tile pair
    cfg3 = dict(B=1, Hq=28, Hk=4, S=4096, D=128, dtype=torch.bfloat16, causal=True, vscale=0.5)
    q, k, v = (t.requires_grad_(True) for t in make_inputs(cfg3, 0, device))
    out = F.attention(q, k, v, True)
    do = torch.randn_like(out)
    ms = time_op(lambda: torch.autograd.grad(out, (q, k, v), do, retain_graph=True), 10, 2)
    pairs = cfg3["S"] * (cfg3["S"] + 1) // 2
    io = (3 * cfg3["Hq"] + 4 * cfg3["Hk"]) * cfg3["S"] * cfg3["D"] * 2 + cfg3["Hq"] * cfg3["S"] * cfg3["D"] * 2
    add("cfg3", "attention_backward", ms, cfg3["Hq"] * cfg3["D"] * 10 * pairs, io,
        "algorithmic work = 5 GEMMs per tile pair; the two-kernel form computes 7 (q.k^T and dout.v^T twice)")
    del q, k, v, out, do

    # score-only operator on cfg2's shape, fp16 scores (the reference's output format)
    q, k, _ = make_inputs(CFG2, 0, device)
    ms = time_op(lambda: F.compute_attention_scores(q, k), 30, 3)
    n = CFG2["Hq"] * CFG2["S"]
    add("cfg2", "compute_attention_scores", ms, 2 * n * CFG2["S"] * CFG2["D"], 2 * n * CFG2["D"] * 2 + n * CFG2["S"] * 2)
    # the headline operator with scores in the input dtype and zeros at hidden entries: what the reference's own
    # kernel writes (attention_with_scores.py:141-152,284); half the score bytes of the fp32 form
    q, k, v = make_inputs(CFG2, 0, device)
    ms = time_op(lambda: F.attention_with_scores(q, k, v, True, scores_dtype=q.dtype, masked_value=0.0), 30, 3)
    flops, nbytes = algorithmic(CFG2, "scores", None)
    add("cfg2", "attention_with_scores (16-bit scores)", ms, flops, nbytes - n * CFG2["S"] * 2)
    del q, k, v

    # decoding: few query rows against 16 384 keys; K/V traffic bounds it.  The G = 4 query heads of a kv head are
    # packed into one query tile (K and V stream once per kv head) and the keys are cut into ranges (split-KV).
    for B in (1, 4):
        for M in (1, 16):
            dec = dict(B=B, Hq=32, Hk=8, D=128, N=16384)
            g = torch.Generator(device=device).manual_seed(M)
            q = torch.randn(dec["B"], dec["Hq"], M, dec["D"], device=device, generator=g).half()
            k = torch.randn(dec["B"], dec["Hk"], dec["N"], dec["D"], device=device, generator=g).half()
            v = torch.randn(dec["B"], dec["Hk"], dec["N"], dec["D"], device=device, generator=g).half()
            kv_bytes = 2 * dec["B"] * dec["Hk"] * dec["N"] * dec["D"] * 2
            flops = 4 * dec["B"] * dec["Hq"] * M * dec["N"] * dec["D"]
            for label, splits in (("attention split-KV", None), ("attention unsplit", 1)):
                ms = time_op(lambda: F.attention(q, k, v, False, kv_splits=splits), 30, 3)
                add(f"decode M={M} N=16384 B={B} Hq=32 Hk=8", label, ms, flops, kv_bytes + 2 * q.numel() * 2)
            del q, k, v
    return rows


CFG4 = dict(B=2, Hq=32, Hk=8, S=4096, D=128, dtype=torch.float16, causal=True, split=3072)
CFG5 = dict(B=4, Hq=32, Hk=8, S=16384, D=128, dtype=torch.bfloat16, causal=False, vdist="uniform", split=12288)


def _max_over_ranks(x, device, world):
    import torch.distributed as dist
    t = torch.tensor([x], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def _all_true(flag, device, world):
    import torch.distributed as dist
    t = torch.tensor([1.0 if flag else 0.0], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item() > 0.5)


def make_unit(cfg, unit, seed, device):
    """q (1,G,S,D), k, v (1,1,S,D) of shard unit `unit` = b*Hk + hk, drawn on the device from seed + unit:
    any rank can build any unit without the others."""
    G, S, D = cfg["Hq"] // cfg["Hk"], cfg["S"], cfg["D"]
    g = torch.Generator(device=device).manual_seed(seed + unit)
    q = torch.randn(1, G, S, D, device=device, generator=g)
    k = torch.randn(1, 1, S, D, device=device, generator=g)
    if cfg.get("vdist") == "uniform":
        v = torch.rand(1, 1, S, D, device=device, generator=g) * 2 - 1
    else:
        v = torch.randn(1, 1, S, D, device=device, generator=g)
    return q.to(cfg["dtype"]), k.to(cfg["dtype"]), v.to(cfg["dtype"])


def _time_calls(fn, iters, warmup, device, world):
    """Mean ms per call over `iters` back-to-back calls, CUDA events, barrier on both sides, max over ranks."""
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    return _max_over_ranks(a.elapsed_time(b) / iters, device, world)


def unit_shard_leg(F, device, rank, world, pk):
    """The partition the path shards by: (batch, kv head) units with their G query heads, dealt to the
    ranks in contiguous blocks (shard.plan_units), no exchange step.  Strong scaling: the whole cfg4 / cfg5
    problem at every N; each rank builds and runs only its units (as a batch of single-kv-head problems).
    Device time, max over ranks; the one-GPU time of all units is measured in the same run on rank 0."""
    from flash_attn_with_score_b200 import shard
    rows = []
    plans = [("cfg4", CFG4, "cross_qk", 20), ("cfg4", CFG4, "cross_softmax", 20), ("cfg5", CFG5, "softmax_col_sum", 3)]
    cache = {}
    for name, cfg, op, iters in plans:
        n_units = cfg["B"] * cfg["Hk"]
        mine = shard.plan_units(n_units, world)[rank]
        G, S, split = cfg["Hq"] // cfg["Hk"], cfg["S"], cfg["split"]
        if name not in cache:
            cache.clear()
            units = [make_unit(cfg, u, 0, device) for u in mine]
            cache[name] = tuple(torch.cat([u[i] for u in units], 0) for i in range(3)) if units else None
        local = cache[name]

        def call(t):
            q, k, v = t
            if op == "cross_qk":
                return F.attention_cross_token_qk_sum(q, k, v, split, cfg["causal"])
            if op == "cross_softmax":
                return F.attention_cross_token_softmax_sum(q, k, v, split, cfg["causal"])
            return F.attention_with_softmax_col_sum(q, k, v, cfg["causal"])

        ms = _time_calls((lambda: call(local)) if local is not None else (lambda: None), iters, 2, device, world)
        # size-independent checks on this rank's units (torch fp64 on the device is the checker here)
        ok = True
        viol = 0.0
        if local is not None:
            q, k, v = local
            out, sums = call(local)
            if op == "cross_qk":  # linear identity: sum_i s_ij = sm_scale * k_j . sum_{i >= split} q_i (j < split <= i)
                qs = q[:, :, split:].double().sum(2).sum(1)  # (units, D): rows >= split, all G heads
                want = torch.einsum("und,ud->un", k[:, 0, :split].double(), qs) / math.sqrt(cfg["D"])
                err = (sums[:, 0].double() - want).abs()
                tol = 1e-3 * want.abs() + 1e-3 * want.pow(2).mean().sqrt()
                viol = float((err - tol).max())
            elif op == "softmax_col_sum":  # every query row spreads a total weight of 1 over the keys
                total = sums.double().sum(-1)
                viol = float(((total - G * S).abs() - 1e-3 * G * S).max())
            else:  # cross_softmax: first query head of the first local unit against plain torch fp32
                s = (q[0, 0, split:].float() @ k[0, 0].float().t()) / math.sqrt(cfg["D"])
                if cfg["causal"]:
                    i = torch.arange(split, S, device=device).unsqueeze(1)
                    j = torch.arange(S, device=device).unsqueeze(0)
                    s = s.masked_fill(j > i, float("-inf"))
                w = torch.softmax(s, -1)[:, :split].double().sum(0)
                _, per_head = F.attention_cross_token_softmax_sum(q[:1], k[:1], v[:1], split, cfg["causal"],
                                                                  per_q_head=True)
                err = (per_head[0, 0].double() - w).abs()
                viol = float((err - (1e-3 * w.abs() + 1e-3 * w.pow(2).mean().sqrt())).max())
            ok = viol <= 0
        ok = _all_true(ok, device, world)
        # all units on one GPU, same run (rank 0)
        t1 = None
        if world > 1 and rank == 0:
            allu = [make_unit(cfg, u, 0, device) for u in range(n_units)]
            full = tuple(torch.cat([u[i] for u in allu], 0) for i in range(3))
            del allu
            for _ in range(2):
                call(full)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                call(full)
            b.record()
            torch.cuda.synchronize()
            t1 = a.elapsed_time(b) / iters
            del full
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        split_arg = split if op != "softmax_col_sum" else None
        flops, _ = algorithmic(cfg, op, split_arg)
        row = {"workload": name, "op": op, "scaling": "strong", "n_gpus": world, "units": n_units,
               "units_per_rank": len(mine), "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
               "frac_of_tensor_peak_all_gpus": flops / (ms * 1e-3) / 1e12 / (world * pk["tensor"]), "parity_ok": ok,
               "parity": {"cross_qk": "linear identity k_j . sum_i q_i", "softmax_col_sum": "mass conservation G*S per unit",
                          "cross_softmax": "one query head against torch fp32 softmax"}[op]}
        if ms >= 2.0:  # milliseconds under the power cap: the sustained matmul peak is the one that applies
            row["frac_of_sustained_peak_all_gpus"] = flops / (ms * 1e-3) / 1e12 / (world * pk["tensor_sustained"])
        if world == 1:
            row["one_gpu_ms"] = ms
        elif t1 is not None:
            row["one_gpu_ms"] = t1
            row["efficiency"] = t1 / (world * ms)
            per_unit = t1 / n_units
            row["limiter"] = ("launch + fixed per-call cost: %.0f us of kernels per rank against ~%.0f us of per-call "
                              "set-up and tail that does not shrink with the unit count"
                              % (per_unit * len(mine) * 1e3, max(0.0, ms - per_unit * len(mine)) * 1e3))
        rows.append(row)
    cache.clear()
    return rows


def query_split_leg(F, device, rank, world, pk):
    """The one path with a collective: the query rows of every head of cfg5 are split over the ranks
    (K/V replicated), each rank runs attention_with_softmax_col_sum on its row window, the fp32
    partial column sums are all-gathered over NCCL and added in rank order on every rank.  Strong
    scaling (the whole cfg5 problem at every N); device time, max over ranks.  The exchange of batch
    element b overlaps the kernels of element b + 1; the exposed part is total - compute-only."""
    import torch.distributed as dist
    from flash_attn_with_score_b200 import shard
    cfg = CFG5
    q, k, v = make_inputs(cfg, 0, device)  # same seed on every rank: identical tensors
    G, S = cfg["Hq"] // cfg["Hk"], cfg["S"]
    steps = 3
    begin, end = shard.plan_query_rows(S, world)[rank]
    res = {}

    def run_overlap():
        res["v"] = shard.query_split(F.attention_with_softmax_col_sum, q, k, v, False, overlap=True)

    def run_serial():
        res["s"] = shard.query_split(F.attention_with_softmax_col_sum, q, k, v, False)

    def run_compute_only():
        for b in range(cfg["B"]):
            F.attention_with_softmax_col_sum(q[b:b + 1], k[b:b + 1], v[b:b + 1], False, q_rows=(begin, end))

    ms = _time_calls(run_overlap, steps, 2, device, world)
    ms_serial = _time_calls(run_serial, steps, 2, device, world)
    ms_compute = _time_calls(run_compute_only, steps, 2, device, world)
    out, sums, rows = res["v"]
    # parity that is not rank-vs-rank: mass conservation per (b, kv head), and one kv head against the unsplit call
    total = sums.double().sum(-1)
    mass_viol = float(((total - G * S).abs() - 1e-3 * G * S).max())
    _, one = F.attention_with_softmax_col_sum(q[:1, :G], k[:1, :1], v[:1, :1], False)
    err = (sums[0, 0].double() - one[0, 0].double()).abs()
    unsplit_viol = float((err - (1e-3 * one[0, 0].double().abs() + 1e-3 * one.double().pow(2).mean().sqrt())).max())
    same_bits = torch.equal(res["s"][1], sums)  # not required: per-element calls may pick another launch shape
    d2 = (res["s"][1].double() - sums.double()).abs()
    forms_viol = float((d2 - (1e-3 * sums.double().abs() + 1e-3 * sums.double().pow(2).mean().sqrt())).max())
    digest = sums.double().sum().reshape(1)
    lo, hi = digest.clone(), digest.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    parity_ok = _all_true(mass_viol <= 0 and unsplit_viol <= 0 and forms_viol <= 0, device, world)
    flops, _ = algorithmic(cfg, "softmax_col_sum", None)
    ms_overlap, ms = ms, min(ms, ms_serial)
    return {"workload": "cfg5", "op": "attention_with_softmax_col_sum", "scaling": "strong", "n_gpus": world,
            "ms_per_step": ms, "ms_per_step_exchange_after_compute": ms_serial,
            "ms_per_step_exchange_overlapped_per_batch_element": ms_overlap, "ms_compute_only": ms_compute,
            "exposed_exchange_ms": max(0.0, ms - ms_compute),  # of the form the headline uses
            "tflops": flops / (ms * 1e-3) / 1e12, "steps": steps, "rows_per_rank": rows[1] - rows[0],
            "collective": "all_gather of the fp32 partial column sums + fixed-order reduce kernel, after the compute "
                          "(whole batch) or per batch element overlapping the next element's kernels; the faster is "
                          "the headline",
            "exchanged_bytes_per_rank": int(sums.numel() * 4 * (world - 1)),
            "sums_identical_on_all_ranks": bool((lo == hi).item()),
            "frac_of_sustained_peak_all_gpus": flops / (ms * 1e-3) / 1e12 / (world * pk["tensor_sustained"]),
            "parity_ok": parity_ok, "mass_conservation_viol": mass_viol, "vs_unsplit_one_kv_head_viol": unsplit_viol,
            "overlapped_vs_serial_viol": forms_viol, "overlapped_equals_serial_bits": bool(same_bits),
            "frac_of_tensor_peak_all_gpus": flops / (ms * 1e-3) / 1e12 / (world * pk["tensor"])}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-ops", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time direct launches instead of CUDA-graph replays")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # stdout carries exactly one JSON line: whatever libraries print there (NCCL's version banner) goes to stderr
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        os.write(json_fd, (json.dumps(obj) + "\n").encode())

    if args.impl == "reference":
        run_reference(args, rank, emit)
        return

    import torch.distributed as dist
    import flash_attn_with_score_b200 as F

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    cfg = CFG2
    pk = peaks()
    flops, nbytes = algorithmic(cfg)
    score_bytes = cfg["B"] * cfg["Hq"] * cfg["S"] * cfg["S"] * 4

    # rotating buffer sets so that every step's reads and writes miss L2
    sets = []
    for i in range(N_SETS):
        q, k, v = make_inputs(cfg, 1000 * rank + i, device)
        out = torch.empty_like(q)
        scores = torch.empty(cfg["B"], cfg["Hq"], cfg["S"], cfg["S"], device=device, dtype=torch.float32)
        sets.append((q, k, v, out, scores))

    def step(i):
        q, k, v, out, scores = sets[i % N_SETS]
        F.attention_with_scores(q, k, v, cfg["causal"], out=out, scores=scores)

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    # The step is launch-bound on the host side (one 42 us kernel per call), so the timed loop replays
    # a CUDA graph that holds one call of the public API per buffer set; steps that do not fill a
    # whole replay are launched directly.
    graph, launches_per_step = None, 1
    if not args.no_graph:
        try:
            cap = torch.cuda.Stream()
            cap.wait_stream(torch.cuda.current_stream())
            n0 = F.launch_count()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=cap):
                for i in range(N_SETS):
                    step(i)
            launches_per_step = max(1, (F.launch_count() - n0) // N_SETS)
            torch.cuda.current_stream().wait_stream(cap)
            g.replay()
            torch.cuda.synchronize()
            graph = g
        except Exception as e:  # capture not possible: time direct launches
            print(f"bench: CUDA graph capture failed ({e}); timing direct launches", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    # warm-up of the timed mechanism itself: the W warm-up steps again, as graph replays
    if graph is not None:
        for _ in range(max(1, -(-args.warmup // N_SETS))):
            graph.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = F.launch_count()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    n_replays = args.steps // N_SETS if graph is not None else 0
    t_start.record()
    for _ in range(n_replays):
        graph.replay()
    for i in range(n_replays * N_SETS, args.steps):
        step(i)
    t_end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches = F.launch_count() - launches0 + n_replays * N_SETS * launches_per_step
    total_ms = t_start.elapsed_time(t_end)
    status = F.device_status()

    # What the timed region wrote, checked outside it: out and scores of the buffer set its last step used
    # (results of the graph replay when a graph was timed) against the CPU oracle.
    parity = check_parity(sets[(args.steps - 1) % N_SETS], cfg) if rank == 0 else None

    # A steadier figure beside the K-step headline: >= 200 graph-replayed launches back to back.
    long_ms = None
    if graph is not None:
        n_long = max(1, -(-200 // N_SETS))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_long):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        long_ms = a.elapsed_time(b) / (n_long * N_SETS)

    # per-step event times of directly launched steps (host launch cost included)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for i in range(args.steps):
        evs[i][0].record()
        step(i)
        evs[i][1].record()
    torch.cuda.synchronize()
    step_event_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)

    # Duration of the kernel itself: the same launches with the stream kept busy (a spin kernel
    # is queued first so the host runs ahead), so that the event pairs bracket the launch and
    # not the host's enqueue latency.
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    torch.cuda.synchronize()
    torch.cuda._sleep(int(4e6 + 1.2e5 * args.steps))
    for i in range(args.steps):
        kev[i][0].record()
        step(i)
        kev[i][1].record()
    torch.cuda.synchronize()
    kern_ms = statistics.mean(a.elapsed_time(b) for a, b in kev)

    t = torch.tensor([total_ms, kern_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, kern_ms = t.tolist()
    ms_per_step = total_ms / args.steps

    # end to end through the public API from pinned host buffers (H2D + op + D2H of out and scores)
    hq, hk, hv = (x.pin_memory() for x in make_inputs(cfg, 7 + rank, None))
    h_out = torch.empty(hq.shape, dtype=hq.dtype).pin_memory()
    h_scores = torch.empty(cfg["B"], cfg["Hq"], cfg["S"], cfg["S"], dtype=torch.float32).pin_memory()
    # Double-buffered: step i's host->device copy, its kernel and its device->host read run on three
    # streams chained by events, so the copies of neighbouring steps overlap (PCIe is full duplex);
    # every step still moves its own inputs in and its own out + scores back.
    s_in, s_op, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_op = [None, None]   # kernel of the step that last used buffer set b
    ev_out = [None, None]  # device->host read of that step

    def e2e_step(i):
        b = i & 1
        dq, dk, dv, dout, dscores = sets[b]
        with torch.cuda.stream(s_in):
            if ev_op[b] is not None:
                s_in.wait_event(ev_op[b])  # the inputs of set b are free once its last kernel ran
            dq.copy_(hq, non_blocking=True)
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
            ev_in = s_in.record_event()
        with torch.cuda.stream(s_op):
            s_op.wait_event(ev_in)
            if ev_out[b] is not None:
                s_op.wait_event(ev_out[b])  # the outputs of set b have been read back
            F.attention_with_scores(dq, dk, dv, cfg["causal"], out=dout, scores=dscores)
            ev_op[b] = s_op.record_event()
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_op[b])
            h_out.copy_(dout, non_blocking=True)
            h_scores.copy_(dscores, non_blocking=True)
            ev_out[b] = s_out.record_event()

    e2e_steps = max(3, min(args.steps, 10))
    for i in range(2):
        e2e_step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s3 in (s_in, s_op, s_out):
        s3.wait_event(e0)
    for i in range(e2e_steps):
        e2e_step(i)
    cur = torch.cuda.current_stream()
    cur.wait_event(ev_out[0])
    cur.wait_event(ev_out[1])
    e1.record()
    torch.cuda.synchronize()
    te = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = te.item() / e2e_steps
    # the sampler ran through the timed steps, the kernel-duration leg and the end-to-end leg
    clocks = sampler.stop() if rank == 0 else None
    h2d = sum(x.numel() * x.element_size() for x in (hq, hk, hv))
    d2h = h_out.numel() * h_out.element_size() + h_scores.numel() * 4

    # bare copies of the same byte counts on the same streams, all ranks at once: the ceiling of the e2e figure
    def copy_only_step(i):
        bset = i & 1
        dq, dk, dv, dout, dscores = sets[bset]
        with torch.cuda.stream(s_in):
            dq.copy_(hq, non_blocking=True)
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
        with torch.cuda.stream(s_out):
            h_out.copy_(dout, non_blocking=True)
            h_scores.copy_(dscores, non_blocking=True)

    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    s_in.wait_event(c0)
    s_out.wait_event(c0)
    for i in range(e2e_steps):
        copy_only_step(i)
    cur.wait_stream(s_in)
    cur.wait_stream(s_out)
    c1.record()
    torch.cuda.synchronize()
    copy_only_ms = _max_over_ranks(c0.elapsed_time(c1) / e2e_steps, device, world)

    qsplit = ushard = None
    if not args.no_ops:
        ushard = unit_shard_leg(F, device, rank, world, pk)
        if world > 1:
            qsplit = query_split_leg(F, device, rank, world, pk)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # Average duration of one launch.  With the graph the timed region is K launches back to back with no
    # host in the loop, so total / K is the launch duration plus the gap to the next launch; a pair of events
    # around a single launch (kernel_event_ms) adds the cost of the two event records to a 40 us kernel.
    if graph is not None:
        launch_ms = ms_per_step
        launch_timing = ("CUDA events around the K graph-replayed launches of the timed region on the launching "
                         "stream, divided by K (launch gaps included)")
    else:
        launch_ms = kern_ms
        launch_timing = "CUDA events around each launch on the launching stream, stream kept busy"
    line = {
        "metric": "attention_with_scores score-write rate", "value": world * score_bytes / (ms_per_step * 1e-3) / 1e9,
        "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "cfg2", "op": "attention_with_scores", "B": 1, "Hq": 32, "Hk": 32, "S": 1024,
                   "D": 128, "causal": True, "scores": "fp32, -inf at hidden entries",
                   "per_gpu_units": 32, "l2": f"{N_SETS} rotating buffer sets (>126 MB L2)",
                   "launch": (f"CUDA graph of {N_SETS} API calls, replayed" if graph is not None else "direct")},
        "tflops": world * flops / (ms_per_step * 1e-3) / 1e12,
        "roofline": {"bound": "hbm", "achieved": nbytes / (launch_ms * 1e-3) / 1e9, "peak": pk["hbm"],
                     "unit": "GB/s", "frac": nbytes / (launch_ms * 1e-3) / 1e9 / pk["hbm"], "traffic": None,
                     "peak_source": pk["src"], "kernel": "tc_fwd_kernel<half,128> (scores hook)",
                     "algorithmic_bytes": nbytes, "kernel_ms": launch_ms, "kernel_ms_long": long_ms,
                     "frac_long": (nbytes / (long_ms * 1e-3) / 1e9 / pk["hbm"]) if long_ms else None,
                     "kernel_event_ms": kern_ms, "frac_event": nbytes / (kern_ms * 1e-3) / 1e9 / pk["hbm"],
                     "step_event_ms": step_event_ms, "timing": launch_timing},
        "e2e": {"value": world * score_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "copy_only_ms": copy_only_ms,
                "limiter": "host link: %.0f %% of the step is the bare H2D + D2H copies of the same bytes "
                           "(all ranks copying at once)" % (100.0 * copy_only_ms / e2e_ms),
                "pipeline": "two buffer sets; H2D, kernel and D2H of neighbouring steps overlap on three streams"},
        "gpu_launches": launches, "backend": F.last_backend(), "device_status": status, "clocks": clocks,
        "parity": parity,
    }
    line["roofline"]["traffic"] = NCU_TRAFFIC_BYTES_PER_LAUNCH
    if ushard is not None:
        line["unit_shard"] = ushard
    if qsplit is not None:
        line["query_split"] = qsplit
    if world == 1 and not args.no_cpu:
        ts = cpu_reference_time(cfg, 5)
        sec = statistics.median(ts)
        cores = torch.get_num_threads()
        line["cpu_baseline"] = {"value": score_bytes / sec / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                                "ms": sec * 1e3,
                                "sample": f"whole cfg2 problem, median of 5 calls of the naive PyTorch path "
                                          f"(oracle port), {cores} threads of {os.cpu_count()} logical CPUs"}
    if world == 1 and not args.no_ops:
        ops_sampler = ClockSampler(local_rank)
        ops_sampler.start()
        try:
            line["ops"] = ops_table(F, device, pk)
        except Exception as e:  # keep the headline line even if a side measurement fails
            line["ops_error"] = repr(e)
        line["ops_clocks"] = ops_sampler.stop()
    emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
