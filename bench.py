#!/usr/bin/env python
"""Benchmark of the shared-KV causal-window hot path (forward + all five gradients).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--window 128]

Workload (the shared-KV configuration the headline metric is quoted on): BF16, one
shared KV head, 8 query heads, D = 128, batch 4, N = 8192, causal window 128;
Q/R/S/Vr/Vs ~ N(0,1)/sqrt(128) from seed 3, dY ~ N(0,1).  A step is one forward
plus one backward over that batch.

One GPU: that problem on the one device (`value`, device-timed with the inputs
resident), the same through the public operator with pinned host buffers (`e2e`),
the window sweep 16/32/64, the long-sequence problem B1 N131072 (`rows`), the
secondary configurations, the reference's own kernels on the same device (`ref_gpu`)
and the CPU restatement on the host cores (`cpu_baseline`).

N > 1 GPUs (one process per GPU, launched by torch.distributed.run): the SAME problem
split by (batch, head) over the ranks -- batches over batch shards, the query heads of
a batch shard over the ranks of its group, whose FP32 key-gradient partials are summed
with NCCL all-reduces (`"scaling": "strong"`, total work fixed).  The line also carries
`rows` (the long sequence row-sharded with a 128-row key halo and the halo key gradients
handed back) and `replicas` (every rank its own copy of the problem, no collective).

Every timing is preceded by a gate on the tensors about to be timed: a slice of the
results against the FP64 CPU oracle with the reference's tolerances and a repeat-call
bit-equality check; a failed gate prints no value.

Algorithmic FLOPs per step = 16 * D * T with T = B * Hq * sum_i min(i+1, w)^2
(forward 4*D*T: score and value contraction; backward 12*D*T: six contractions).
`--impl reference` times the CPU restatement of the reference's naive path
(oracle/triplet_oracle.py) on the host cores instead.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

B, HQ, HKV, N, D = 4, 8, 1, 8192, 128
N_LONG = 131072
METRIC = "fwd+bwd TFLOP/s, shared-KV causal w=128 d=128"
SEED = 3


def triplets(batch, heads, n, w):
    full = max(0, n - w + 1) * w * w
    ramp = sum(min(i + 1, w) ** 2 for i in range(min(n, w - 1)))
    return batch * heads * (full + ramp)


def measured_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("bf16_tflops", 1590.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = sorted(sm)[len(sm) // 2:]            # the idle samples before/after the region sit in the lower half
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def draw_shared(batch, n, seed, d=D, hq=None):
    """(Q, R, S, Vr, Vs, dY) on the CPU in the reference's draw order (tests/test_single_gather_shared.py:45-54)."""
    hq = hq or HQ
    g = torch.Generator(device="cpu").manual_seed(seed)
    s = 1.0 / math.sqrt(d)
    Q = (torch.randn(batch, hq, n, d, generator=g) * s).to(torch.bfloat16)
    kv = [(torch.randn(batch, HKV, n, d, generator=g) * s).to(torch.bfloat16) for _ in range(4)]
    dY = torch.randn(batch, hq, n, d, generator=g).to(torch.bfloat16)
    return (Q, *kv, dY)


# --------------------------------------------------------------------------- CPU arm (oracle port)

def cpu_sample(window, queries=4096, batch=1):
    """fwd+bwd of the banded FP32 restatement on `queries` interior queries of one
    batch (all 8 heads, full window) with every host thread.  Returns (TFLOP/s, seconds, cores)."""
    from oracle import triplet_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = queries + window - 1
    n += (-n) % 16
    Q, R, S, Vr, Vs, dY = draw_shared(batch, n, SEED)
    q_begin = n - queries
    t0 = time.perf_counter()
    O.single_gather_banded(Q, R, S, Vr, Vs, window=window, dY=dY, chunk=32, q_begin=q_begin, dtype=torch.float32)
    dt = time.perf_counter() - t0
    flops = 16 * D * batch * HQ * sum(min(i + 1, window) ** 2 for i in range(q_begin, n))
    return flops / dt / 1e12, dt, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    for _ in range(args.warmup):
        cpu_sample(args.window, queries=256)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        v, dt, cores = cpu_sample(args.window, queries=args.cpu_queries)
        vals.append(v)
    total = time.perf_counter() - t0
    value = statistics.mean(vals)
    sample = (f"banded FP32 torch restatement, 1 batch x 8 heads x {args.cpu_queries} interior queries "
              f"(full window {args.window}) per step")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / max(1, args.steps),
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"shared-KV B{B} Hq{HQ} Hkv{HKV} N{N} D{D} causal window {args.window}",
                   "note": "each step is a bounded sample of that workload on the host cores"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# --------------------------------------------------------------------------- common GPU plumbing

class Ctx:
    def __init__(self, need_group):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the sm_100a kernels have no CPU path")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.grouped = self.world > 1 or need_group
        if self.grouped:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
            dist.init_process_group("nccl", rank=self.rank, world_size=self.world, device_id=self.dev)
        from att3ntion_b200 import _cabi, _cuda_kernels
        self.cabi, self.ck, self.lib = _cabi, _cuda_kernels, _cabi.lib

    def barrier(self):
        if self.grouped and self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = torch.tensor([x], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.item()

    def all_ok(self, ok: bool) -> bool:
        if self.world == 1:
            return ok
        t = torch.tensor([1.0 if ok else 0.0], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return t.item() > 0.5

    def launches(self) -> int:
        return sum(self.lib.att3_launch_count(i) for i in range(4))

    def timed(self, step, steps, warmup):
        """`warmup` untimed steps, then exactly `steps` steps between two CUDA events, bracketed by a
        barrier + synchronize on both sides; milliseconds per step, maximum over the ranks."""
        for _ in range(warmup):
            step()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1)) / steps

    def close(self):
        if self.grouped:
            self.dist.destroy_process_group()


def gate_single_device(ck, host, dev_t, w, b, lo, hi, heads_all=True):
    """Gate before timing (benchmarks/bench_single_gather.py:887-961): forward + backward on the tensors
    about to be timed, a slice against the FP64 oracle (Y, LSE, dQ, complete key-gradient rows) and a
    repeated backward that must be bit-identical.  Returns the gate record."""
    from oracle import triplet_oracle as O
    Q, R, S, Vr, Vs, dY = dev_t
    rec = {"checked": [], "max_rel_l2": None, "passed": False,
           "slice": f"batch {b}, queries [{lo},{hi}) vs banded FP64 oracle; repeat backward bit-equal"}
    try:
        Y, m, l = ck.sg_forward_raw(Q, R, S, Vr, Vs, None, w)
        g1 = ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w)
        g2 = ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w)
        ck.device_status()
        got = {"Y": Y, "m": m, "l": l, "dQ": g1[0], "dR": g1[1], "dS": g1[2], "dVr": g1[3], "dVs": g1[4]}
        rels = O.slice_gate(host, got, w, b, lo, hi)
        assert all(torch.equal(a, c) for a, c in zip(g1, g2)), "repeated backward differs"
        rec.update(checked=sorted(rels) + ["LSE", "repeat"], max_rel_l2=max(rels.values()), passed=True)
    except AssertionError as e:
        rec["error"] = str(e)
    return rec


def e2e_loop(ctx, host_in, host_out, run_step, steps):
    """End to end with host buffers: every step copies its own inputs host -> device and its own results
    device -> host; the copies run on two side streams, so the input copy of step k+1 and the result copy of
    step k-1 overlap the kernels of step k (double-buffered device inputs), as an input pipeline in front of
    a training step would.  `run_step(dev_inputs) -> list of result tensors` (in host_out order).
    Returns milliseconds per step (maximum over ranks)."""
    dev = ctx.dev
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)
    dev_in = [[torch.empty_like(t, device=dev) for t in host_in] for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]                       # results of the last two steps stay alive while they are copied out

    def prefetch(k):
        slot = k & 1
        with torch.cuda.stream(s_in):
            if k >= 2:
                s_in.wait_event(consumed[slot])          # the kernels of step k-2 have read this buffer
            for dst, src in zip(dev_in[slot], host_in):
                dst.copy_(src, non_blocking=True)
            in_ready[slot].record(s_in)

    def one(k):
        slot = k & 1
        main.wait_event(in_ready[slot])
        results = run_step(dev_in[slot])
        consumed[slot].record(main)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for dst, src in zip(host_out, results):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)
        keep[slot] = results

    def run(n):
        prefetch(0)
        for k in range(n):
            if k + 1 < n:
                prefetch(k + 1)
            one(k)
        main.wait_stream(s_out)                          # the last results are on the host when the clock stops

    run(2)
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(steps)
    e1.record()
    ctx.barrier()
    return ctx.max_over_ranks(e0.elapsed_time(e1)) / steps


def kernel_times(lib):
    out = {}
    for k, name in enumerate(["sg_ring_fwd", "sg_ring_bwd", "sg_bwd_reduce"]):
        tot, cnt = C.c_double(), C.c_ulonglong()
        lib.att3_timing_read(k, C.byref(tot), C.byref(cnt))
        out[name] = (tot.value, cnt.value)
    return out


# DRAM bytes (read + write) of one sg_ring_bwd_kernel launch, from an ncu capture of the kernels at
# B4 Hq8 Hkv1 N4096 D128 w128: 123.1 MB (key side S + dQ) and 95.8 MB (key side R), i.e. 6683 bytes
# per (batch, query) on average over the two launches of a step.  The traffic is per-row streaming
# (Q, dY, Y rows, key rows, FP32 partial rows), so it scales with B*N; other head counts, head sizes
# or windows have not been captured (None).
def traffic_bytes_per_launch(batch, hq, hkv, n, d, w):
    if (hq, hkv, d, w) == (8, 1, 128, 128):
        return 6683 * batch * n
    return None


# --------------------------------------------------------------------------- one GPU: the headline line

def window_sweep(ctx, host, dev_t, steps):
    """Windows 16/32/64 of the same problem: gate, then a short timed loop each."""
    out = {}
    burst, _, _ = measured_peaks()
    Q, R, S, Vr, Vs, dY = dev_t
    for w in (16, 32, 64):
        gate = gate_single_device(ctx.ck, host, dev_t, w, B // 2, N // 2 - 96, N // 2 + 96)
        rec = {"gate": gate}
        if gate["passed"]:
            def step():
                Y, m, l = ctx.ck.sg_forward_raw(Q, R, S, Vr, Vs, None, w)
                ctx.ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w)
            ms = ctx.timed(step, steps, 3)
            tf = 16 * D * triplets(B, HQ, N, w) / (ms * 1e-3) / 1e12
            rec.update(ms_per_step=ms, tflops=tf, frac_of_burst_peak=tf / burst)
        out[str(w)] = rec
    ctx.ck.device_status()
    return out


def long_sequence_single(ctx, steps):
    """B1 Hq8 Hkv1 N131072 D128 w128 on one device (the 1-GPU point of the row-sharded curve).  Gate: a slice
    that straddles row 16384 (a shard boundary of the 8-GPU split) against the oracle."""
    host = draw_shared(1, N_LONG, 4)
    dev_t = [t.to(ctx.dev) for t in host]
    gate = gate_single_device(ctx.ck, host, dev_t, 128, 0, 16384 - 96, 16384 + 96)
    rec = {"workload": f"shared-KV B1 Hq{HQ} Hkv1 N{N_LONG} D{D} causal window 128, seed 4", "n_gpus": 1, "gate": gate}
    if gate["passed"]:
        Q, R, S, Vr, Vs, dY = dev_t

        def step():
            Y, m, l = ctx.ck.sg_forward_raw(Q, R, S, Vr, Vs, None, 128)
            ctx.ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, 128)
        ms = ctx.timed(step, steps, 3)
        rec.update(ms_per_step=ms, value=16 * D * triplets(1, HQ, N_LONG, 128) / (ms * 1e-3) / 1e12, unit="TFLOP/s")
    ctx.ck.device_status()
    return rec


def run_single(args):
    ctx = Ctx(need_group=False)
    lib, ck = ctx.lib, ctx.ck
    from att3ntion_b200 import single_gather_shared_attention
    ctx.cabi.check(lib.att3_sg_set_query_block(args.fwd_block, args.bwd_block))
    w = args.window
    host = draw_shared(B, N, SEED)
    host_in = [t.pin_memory() for t in host]
    dev_t = [t.to(ctx.dev, non_blocking=True) for t in host_in]
    Q, R, S, Vr, Vs, dY = dev_t
    torch.cuda.synchronize()
    flops_step = 16 * D * triplets(B, HQ, N, w)

    def step():
        Y, m, l = ck.sg_forward_raw(Q, R, S, Vr, Vs, None, w, precise=args.precise)
        return Y, ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w, precise=args.precise)

    if args.profile:
        # kernel-only run for profiler captures: exact warm-up count, no gate, no e2e, no CPU leg
        for _ in range(args.warmup):
            step()
        lib.att3_timing_enable(1)
        kernel_times(lib)
        ms = ctx.timed(step, args.steps, 0)
        kt = kernel_times(lib)
        lib.att3_timing_enable(0)
        ck.device_status()
        print(json.dumps({"profile_run": True, "ms_per_step": ms, "value": flops_step / (ms * 1e-3) / 1e12,
                          "kernel_ms": {k: (v[0] / v[1] if v[1] else None) for k, v in kt.items()}}))
        return

    gate = gate_single_device(ck, host, dev_t, w, B // 2, N // 2 - 96, N // 2 + 96)
    if not gate["passed"]:
        print(json.dumps({"metric": METRIC, "value": None, "unit": "TFLOP/s", "n_gpus": 1, "gate": gate,
                          "error": "the gate failed on the tensors about to be timed; no timing is published"}))
        raise SystemExit(1)

    sampler = ClockSampler(ctx.local)
    sampler.__enter__()                      # nvidia-smi needs a moment to start: begin before the warm-up
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    lib.att3_timing_enable(1)
    kernel_times(lib)                        # drop anything recorded so far
    l0 = ctx.launches()
    ms_step = ctx.timed(step, args.steps, 0)
    launches = ctx.launches() - l0
    ktime = kernel_times(lib)
    lib.att3_timing_enable(0)
    ck.device_status()
    value = flops_step / (ms_step * 1e-3) / 1e12

    # --- end to end through the public operator with host buffers (pinned), copies inside the timed region
    host_out = [torch.empty_like(t).pin_memory() for t in (host[0], host[0], *host[1:5])]   # Y, dQ, dR, dS, dVr, dVs
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    def api_step(dev_in):
        q, r, s, vr, vs, dy = dev_in
        leaves = [t.detach().requires_grad_(True) for t in (q, r, s, vr, vs)]
        y = single_gather_shared_attention(*leaves, None, window=w)
        y.backward(dy)
        return [y.detach()] + [leaf.grad for leaf in leaves]

    e2e_steps = max(2, min(args.steps, 20))
    e2e_ms = e2e_loop(ctx, host_in, host_out, api_step, e2e_steps)
    e2e_value = flops_step / (e2e_ms * 1e-3) / 1e12
    sampler.__exit__()                       # the samples cover the warm-up, the timed loop and the end-to-end loop

    burst, sustained, src = measured_peaks()
    bwd_ms, bwd_n = ktime["sg_ring_bwd"]
    # dominant kernel: one backward pass launch produces one key side's gradients (and dQ once),
    # half of the backward's 12*D*T algorithmic FLOPs
    flops_launch = 6 * D * triplets(B, HQ, N, w)
    achieved = flops_launch / (bwd_ms / max(1, bwd_n) * 1e-3) / 1e12 if bwd_n else None
    roofline = {"bound": "tensor", "kernel": "sg_ring_bwd_kernel<128>", "achieved": achieved, "peak": burst,
                "unit": "TFLOP/s", "frac": (achieved / burst) if achieved else None,
                "peak_source": f"{src} bf16_tflops (burst cuBLAS figure; the timed region runs at full clock)",
                "frac_of_sustained_peak": (achieved / sustained) if achieved else None,
                "traffic": traffic_bytes_per_launch(B, HQ, HKV, N, D, w),
                "kernel_ms": {k: (v[0] / v[1] if v[1] else None) for k, v in ktime.items()},
                "step_frac_of_burst_peak": value / burst}
    out = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"shared-KV B{B} Hq{HQ} Hkv{HKV} N{N} D{D} causal window {w}, fwd + 5 gradients",
                   "per_gpu_batch": B, "parallelism": "one device",
                   "l2": "inputs+outputs 0.5 GB per step exceed the 126 MB L2; no explicit flush",
                   "flops_per_step": flops_step},
        "gate": gate,
        "clocks": sampler.summary(),
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps,
                "copies": "every step's inputs and results cross PCIe inside the timed region, on two side "
                          "streams that overlap the neighbouring steps' kernels"},
        "gpu_launches": int(launches),
        "roofline": roofline,
    }
    if not args.quick:
        short = max(3, min(args.steps, 10))
        out["windows"] = window_sweep(ctx, host, dev_t, short)
        out["rows"] = long_sequence_single(ctx, max(3, min(args.steps, 5)))
        torch.cuda.empty_cache()
        out["secondary"] = secondary_configs(ctx, short)
        out["ref_gpu"] = reference_gpu_arm([128, 64, 32, 16])
    if not args.no_cpu:
        cpu_v, cpu_dt, cores = cpu_sample(w, queries=args.cpu_queries)
        out["cpu_baseline"] = {"value": cpu_v, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                               "sample": f"banded FP32 torch restatement of the naive path, 1 batch x 8 heads x "
                                         f"{args.cpu_queries} interior queries, {cpu_dt:.1f} s"}
    print(json.dumps(out))


# --------------------------------------------------------------------------- secondary configurations

def secondary_configs(ctx, reps):
    """C3 = independent-head single gather B4 H8 N2048 D64 w128, seed 2 (16*D*T FLOPs); C2 = three-gather
    operator B8 H4 N256 D64, seed 1, without mask or scatter (3*(4+14)*D*B*H*N^3 FLOPs, the reference's own
    count), and the same shape with the scatter outputs switched on (time only).  Each is gated on the
    tensors it times: C3 by a slice of two (batch, head) pairs against the banded oracle, C2 by two
    (batch, head) pairs against the dense FP64 three-gather oracle with the reference's tolerances
    (tests/test_kernel_correctness.py:303-361)."""
    from oracle import triplet_oracle as O
    ck, dev = ctx.ck, ctx.dev

    def med(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    out = {}
    # ---- C3
    b3, h3, n3, d3, w3 = 4, 8, 2048, 64, 128
    g = torch.Generator(device="cpu").manual_seed(2)
    h5 = [(torch.randn(b3, h3, n3, d3, generator=g) / math.sqrt(d3)).to(torch.bfloat16) for _ in range(5)]
    hdy = torch.randn(b3, h3, n3, d3, generator=g).to(torch.bfloat16)
    t5 = [t.to(dev) for t in h5]
    dy = hdy.to(dev)
    rec = {"gate": {"passed": False}}
    try:
        Y, m, l = ck.sg_forward_raw(*t5, None, w3)
        gr = ck.sg_backward_raw(dy, *t5, Y, m, l, None, w3)
        ck.device_status()
        rels = {}
        for (b, h) in ((1, 2), (3, 7)):
            sel = lambda t: t[b:b + 1, h:h + 1]
            got = {"Y": sel(Y), "m": m[b:b + 1, h:h + 1], "l": l[b:b + 1, h:h + 1], "dQ": sel(gr[0]),
                   "dR": sel(gr[1]), "dS": sel(gr[2]), "dVr": sel(gr[3]), "dVs": sel(gr[4])}
            r = O.slice_gate(tuple(sel(t) for t in (*h5, hdy)), got, w3, 0, 1024 - 96, 1024 + 96)
            rels.update({f"{k}[{b},{h}]": v for k, v in r.items()})
        rec["gate"] = {"passed": True, "max_rel_l2": max(rels.values()), "checked": "(b,h) = (1,2), (3,7), queries [928,1120)"}
    except AssertionError as e:
        rec["gate"]["error"] = str(e)
    if rec["gate"]["passed"]:
        def c3():
            Y, m, l = ck.sg_forward_raw(*t5, None, w3)
            ck.sg_backward_raw(dy, *t5, Y, m, l, None, w3)
        ms = med(c3)
        rec.update(ms=ms, tflops=16 * d3 * triplets(b3, h3, n3, w3) / ms / 1e9)
    out["C3 single gather B4 H8 N2048 D64 w128"] = rec

    # ---- C2
    g = torch.Generator(device="cpu").manual_seed(1)
    b2, h2, n2, d2 = 8, 4, 256, 64
    hins = [(torch.randn(b2, h2, n2, d2, generator=g) * (0.5 if k < 3 else 1.0)).to(torch.bfloat16) for k in range(9)]
    for k in (4, 6, 8):
        hins[k].zero_()
    hcot = [torch.randn(b2, h2, n2, d2, generator=g).to(torch.bfloat16) for _ in range(3)]
    ins = [t.to(dev) for t in hins]
    cot = [t.to(dev) for t in hcot] + [torch.zeros(b2, h2, n2, d2, dtype=torch.bfloat16, device=dev) for _ in range(3)]
    rec = {"gate": {"passed": False}}
    try:
        o = ck.forward(*ins, 0.0, -1, -1, -1, None, 0)
        gr = ck.backward(*cot, *ins, *o[6:12], 0.0, None, o[0], o[1], o[2])
        ck.device_status()
        worst = 0.0
        for (b, h) in ((0, 0), (5, 3)):
            sub = [t[b:b + 1, h:h + 1] for t in hins]
            ref_out, _ = O.hypergraph_dense(*sub, scatter=False)
            ref_gr = O.hypergraph_grads(sub, [t[b:b + 1, h:h + 1] for t in hcot] + [None] * 3, scatter=False)
            pairs = [(f"output {k}", o[k], ref_out[k], 5e-2, 5e-2) for k in range(3)]
            pairs += [(f"gradient {k}", gr[k], ref_gr[k], rt, at)
                      for k, (rt, at) in zip((0, 1, 2, 3, 5, 7), [(5e-2, 1e-1)] * 3 + [(2e-2, 2e-2)] * 3)]
            for name, a, r, rt, at in pairs:        # |a - r| <= atol * max(1, max|r|) + rtol * |r|, as torch.allclose
                a, r = a[b:b + 1, h:h + 1].float().cpu(), r.float()
                err = (a - r).abs()
                lim = at * max(1.0, r.abs().max().item()) + rt * r.abs()
                assert (err <= lim).all(), f"C2 {name} at (b,h)=({b},{h}): {(err - lim).max().item()} over the limit"
                worst = max(worst, (err / lim).max().item())
        rec["gate"] = {"passed": True, "worst_err_over_tol": worst, "checked": "(b,h) = (0,0), (5,3): 3 outputs, 6 gradients"}
    except AssertionError as e:
        rec["gate"]["error"] = str(e)
    if rec["gate"]["passed"]:
        def c2():
            o = ck.forward(*ins, 0.0, -1, -1, -1, None, 0)
            ck.backward(*cot, *ins, *o[6:12], 0.0, None, o[0], o[1], o[2])
        ms = med(c2)
        rec.update(ms=ms, tflops=3 * (4 + 14) * d2 * b2 * h2 * n2 ** 3 / ms / 1e9)
        # the same shape with the second value tensors in use (module option scatter=True): no FLOP model is
        # published for that part, so only the time is reported
        ins2 = [t.clone() for t in ins]
        for k in (4, 6, 8):
            ins2[k] = torch.randn(b2, h2, n2, d2, generator=g).to(torch.bfloat16).to(dev)
        cot2 = cot[:3] + [torch.randn(b2, h2, n2, d2, generator=g).to(torch.bfloat16).to(dev) for _ in range(3)]

        def c2s():
            o = ck.forward(*ins2, 0.0, -1, -1, -1, None, 0)
            ck.backward(*cot2, *ins2, *o[6:12], 0.0, None, o[0], o[1], o[2])
        rec["ms_with_scatter_outputs"] = med(c2s)
    out["C2 three-gather B8 H4 N256 D64"] = rec
    ck.device_status()
    return out


def run_other(args):
    ctx = Ctx(need_group=False)
    print(json.dumps({"secondary_configs": secondary_configs(ctx, max(3, min(args.steps, 20))), "data": "synthetic"}))


# --------------------------------------------------------------------------- the reference's own kernels on this GPU

def reference_gpu_arm(windows):
    """Times the reference's CUDA kernels (its own sources, compiled for this GPU into baseline/_ref) on the
    headline problem through its binding-level functions with fwd_group=0 / rs_group=0, in a child process
    (its package and torch.library operator names collide with this repository's).  Unavailable when the
    install is absent."""
    ref_dir = REPO / "baseline" / "_ref"
    if not (ref_dir / "att3ntion").is_dir():
        return {"unavailable": "baseline/_ref holds no install of the reference"}
    out = {}
    for w in windows:
        try:
            r = subprocess.run([sys.executable, str(Path(__file__).resolve()), "--refgpu-child", "--window", str(w)],
                               capture_output=True, text=True, timeout=600)
            line = [x for x in r.stdout.splitlines() if x.startswith("{")]
            out[str(w)] = json.loads(line[-1]) if (r.returncode == 0 and line) else \
                {"unavailable": f"child exited {r.returncode}: {(r.stderr or r.stdout).strip().splitlines()[-1:]}"}
        except subprocess.TimeoutExpired:
            out[str(w)] = {"unavailable": "the reference kernels did not finish within 600 s"}
        if "unavailable" in out[str(w)]:
            break                      # a case that failed is not tried again with another window
    return out


def refgpu_child(args):
    """Runs inside the child: the reference's kernels and this repository's on identical seeded inputs."""
    sys.path.insert(0, str(REPO / "baseline" / "_ref"))
    import att3ntion._cuda_kernels as rck          # the reference's pybind module
    from att3ntion_b200 import _cuda_kernels as ck  # binding level only: no operator registration
    from oracle import triplet_oracle as O
    w = args.window
    dev = torch.device("cuda", 0)
    host = draw_shared(B, N, SEED)
    Q, R, S, Vr, Vs, dY = (t.to(dev) for t in host)
    i = torch.arange(N, device=dev)
    mask = ((i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - w))[None].expand(B, -1, -1).contiguous()

    def ev(fn, reps):
        for _ in range(2):
            fn()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); r = fn(); b.record(); torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts), r

    fwd_ms, (Y, m, l) = ev(lambda: rck.single_gather_shared_forward(Q, R, S, Vr, Vs, mask, w, 0), 7)
    bwd_ms, grads = ev(lambda: rck.single_gather_shared_backward(dY, Q, R, S, Vr, Vs, Y, m, l, mask, w, 0), 7)
    Yo, mo, lo_ = ck.sg_forward_raw(Q, R, S, Vr, Vs, None, w)
    go = ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Yo, mo, lo_, None, w)
    ck.device_status()
    rel = {"Y": O.errors(Yo, Y)[0]}
    rel["LSE_max_abs"] = (O.lse_from_ml(mo, lo_) - O.lse_from_ml(m, l)).abs().max().item()
    for name, a, r in zip(["dQ", "dR", "dS", "dVr", "dVs"], go, grads):
        rel[name] = O.errors(a, r)[0]
    step = fwd_ms + bwd_ms
    print(json.dumps({"fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "step_ms": step,
                      "tflops": 16 * D * triplets(B, HQ, N, w) / step / 1e9,
                      "call": "single_gather_shared_forward/backward(fwd_group=0, rs_group=0), window mask built once "
                              "outside the timed region, median of 7",
                      "dispatch": {k: v for k, v in rck.sg_dispatch().items() if "shared" in k},
                      "rel_l2_ours_vs_reference_kernels": rel}))


# --------------------------------------------------------------------------- N GPUs: the (batch, head) partition

def plan_heads(world, batch, head_groups):
    """(batch shards, ranks per shard).  Default: batches first (no communication between batch shards), the
    query heads of a batch shard over what is left."""
    hg = head_groups
    if not hg:
        bs = max(d for d in range(1, world + 1) if world % d == 0 and d <= batch)
        hg = world // bs
    if world % hg or HQ % hg:
        raise SystemExit(f"bench.py: {world} ranks do not split into head groups of {hg}")
    return world // hg, hg


def heads_problem(ctx, args):
    from att3ntion_b200._dist import HeadShardedGather, shard_batch
    dist = ctx.dist
    n, w, Bt = args.seq_len, args.window, args.batch
    bshards, hg = plan_heads(ctx.world, Bt, args.head_groups)
    brank, hrank = ctx.rank // hg, ctx.rank % hg
    groups = [dist.new_group(list(range(b * hg, (b + 1) * hg))) for b in range(bshards)]
    op = HeadShardedGather(w, group=groups[brank])
    batches = list(shard_batch(Bt, bshards, brank))
    heads = HeadShardedGather.local_heads(HQ, 1, hg, hrank)
    host = draw_shared(Bt, n, SEED)
    mine = [host[0][batches][:, heads].contiguous()] + [t[batches].contiguous() for t in host[1:5]] + \
           [host[5][batches][:, heads].contiguous()]
    return op, host, mine, batches, heads, bshards, hg


def run_scale(args):
    """Default for N > 1: the headline problem split by (batch, head), plus the row-sharded long sequence and
    the replica run in the same line."""
    ctx = Ctx(need_group=True)
    lib, ck, dist = ctx.lib, ctx.ck, ctx.dist
    from oracle import triplet_oracle as O
    w = args.window
    op, host, mine, batches, heads, bshards, hg = heads_problem(ctx, args)
    host_in = [t.pin_memory() for t in mine]
    dev_t = [t.to(ctx.dev, non_blocking=True) for t in host_in]
    torch.cuda.synchronize()
    flops_step = 16 * D * triplets(args.batch, HQ, args.seq_len, w)

    def run_step(t):
        q, r, s, vr, vs, dy = t
        y = op.forward(q, r, s, vr, vs)
        dq, dr, ds, dvr, dvs = op.backward(dy)
        return [y, dq, dr, ds, dvr, dvs]

    # gate on every rank's own slice (its first batch, its heads); every rank must pass
    n = args.seq_len
    ok, rec = True, {"passed": False}
    try:
        y, dq, dr, ds, dvr, dvs = run_step(dev_t)
        again = run_step(dev_t)
        ck.device_status()
        Ystat = op._saved
        got = {"Y": y, "m": Ystat[6], "l": Ystat[7], "dQ": dq, "dR": dr, "dS": ds, "dVr": dvr, "dVs": dvs}
        sub_host = tuple(t[batches] for t in host)
        rels = O.slice_gate(sub_host, got, w, 0, n // 2 - 96, n // 2 + 96, heads=heads)
        assert all(torch.equal(a, b_) for a, b_ in zip([y, dq, dr, ds, dvr, dvs], again)), "repeated step differs"
        rec = {"passed": True, "max_rel_l2": max(rels.values()), "checked": sorted(rels) + ["LSE", "repeat"],
               "slice": f"every rank: its first batch, its heads, queries [{n // 2 - 96},{n // 2 + 96}) vs banded FP64 "
                        f"oracle (key gradients after the all-reduce); repeat step bit-equal"}
    except AssertionError as e:
        ok, rec = False, {"passed": False, "error": f"rank {ctx.rank}: {e}"}
    if not ctx.all_ok(ok):
        if ctx.rank == 0:
            print(json.dumps({"metric": METRIC, "value": None, "n_gpus": ctx.world, "gate": rec,
                              "error": "the gate failed on some rank; no timing is published"}))
        ctx.close()
        raise SystemExit(1)

    sampler = ClockSampler(ctx.local)
    sampler.__enter__()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        run_step(dev_t)
    l0 = ctx.launches()
    ms_step = ctx.timed(lambda: run_step(dev_t), args.steps, 0)
    launches = ctx.launches() - l0
    ck.device_status()
    value = flops_step / (ms_step * 1e-3) / 1e12

    # end to end: each rank's own inputs host -> device and its results device -> host every step
    host_out = [torch.empty_like(t).pin_memory() for t in (mine[0], mine[0], *mine[1:5])]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)
    e2e_steps = max(2, min(args.steps, 20))
    e2e_ms = e2e_loop(ctx, host_in, host_out, run_step, e2e_steps)
    sampler.__exit__()                       # the samples cover the warm-up, the timed loop and the end-to-end loop
    del dev_t
    torch.cuda.empty_cache()

    rows = rows_measure(ctx, args, max(3, min(args.steps, 10)))
    torch.cuda.empty_cache()
    replicas = replicas_measure(ctx, args, max(3, min(args.steps, 10)))

    if ctx.rank == 0:
        burst, sustained, src = measured_peaks()
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": ctx.world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"shared-KV B{args.batch} Hq{HQ} Hkv{HKV} N{args.seq_len} D{D} causal window {w}, "
                                   f"fwd + 5 gradients, ONE problem over all ranks",
                       "parallelism": f"(batch, head): {bshards} batch shard(s) x {hg} head group(s); FP32 key-gradient "
                                      f"partials all-reduced (NCCL) inside a batch shard, the first key side's while the "
                                      f"second is computed",
                       "allreduce_bytes_per_step_per_rank": (4 * len(batches) * args.seq_len * D * 4) if hg > 1 else 0,
                       "l2": "per-rank inputs+outputs exceed the 126 MB L2 only up to 4 ranks; no explicit flush",
                       "flops_per_step": flops_step},
            "gate": rec, "clocks": sampler.summary(),
            "e2e": {"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d * ctx.world,
                    "d2h_bytes_per_step": d2h * ctx.world, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "copies": "every rank copies its own share of the inputs in and its results out inside the timed "
                              "region, on two side streams that overlap the neighbouring steps' kernels"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": value / ctx.world, "peak": burst, "unit": "TFLOP/s",
                         "frac": value / ctx.world / burst, "peak_source": f"{src} bf16_tflops (burst)",
                         "note": "whole step per GPU (compute + collective), not a single kernel"},
            "rows": rows, "replicas": replicas,
        }))
    ctx.close()


def rows_measure(ctx, args, steps):
    """The long sequence B1 Hq8 N131072 row-sharded over the ranks (strong scaling): 128-row key halo from the
    left neighbour, halo key gradients handed back in FP32.  Gate on every rank with a right neighbour: the
    64 key rows before its shard end (their gradients include the neighbour's hand-back) and the queries there."""
    from att3ntion_b200._dist import RowShardedGather
    from oracle import triplet_oracle as O
    n, w = N_LONG, 128
    op = RowShardedGather(n, w)
    lo, hi = op.plan.lo, op.plan.hi
    host = draw_shared(1, n, 4)
    B1, n_own = 1, hi - lo
    views = op.local_buffers(B1, HQ, 1, D, torch.bfloat16, ctx.dev)
    for v, t in zip(views, host):
        v.copy_(t[:, :, lo:hi])            # the shards are written where the kernels read them: no copies per step
    Q, R, S, Vr, Vs, dY = views
    flops_step = 16 * D * triplets(1, HQ, n, w)

    def step():
        y = op.forward(Q, R, S, Vr, Vs)
        return y, op.backward(dY)

    ok, err = True, None
    try:
        y, (dq, dr, ds, dvr, dvs) = step()
        ctx.ck.device_status()
        if op.plan.right is not None:
            a, c = hi - 64, hi + 128
            sl = slice(a - 127, c)
            ref = O.single_gather_banded(*[t[:, :, sl] for t in host[:5]], window=w, dY=host[5][:, :, sl], q_begin=127,
                                         chunk=32)
            O.check_gate("Y", y[:, :, n_own - 64:].float().cpu(), ref["Y"][:, :, 127:127 + 64])
            O.check_gate("dQ", dq[:, :, n_own - 64:].float().cpu(), ref["dQ"][:, :, 127:127 + 64])
            for name, t in zip(("dR", "dS", "dVr", "dVs"), (dr, ds, dvr, dvs)):
                O.check_gate(name, t[:, :, n_own - 64:].float().cpu(), ref[name][:, :, 127:127 + 64])
    except AssertionError as e:
        ok, err = False, f"rank {ctx.rank}: {e}"
    passed = ctx.all_ok(ok)
    rec = {"workload": f"shared-KV B1 Hq{HQ} Hkv1 N{n} D{D} causal window {w}, seed 4, rows sharded over {ctx.world} "
                       f"GPU(s), 128-row key halo, halo key gradients handed back in FP32",
           "n_gpus": ctx.world, "scaling": "strong", "shards": op.shards,
           "gate": {"passed": passed, "checked": "every rank with a right neighbour: Y, dQ and the four key gradients on "
                                                 "the 64 rows before its shard end vs banded FP64 oracle"}}
    if err:
        rec["gate"]["error"] = err
    if passed:
        l0 = ctx.launches()
        ms = ctx.timed(step, steps, 3)
        rec.update(ms_per_step=ms, value=flops_step / (ms * 1e-3) / 1e12, unit="TFLOP/s",
                   gpu_launches=int(ctx.launches() - l0), steps=steps)
        ctx.ck.device_status()
    return rec


def replicas_measure(ctx, args, steps):
    """Every rank its own copy of the headline problem: no collective on the data path (weak scaling)."""
    w = args.window
    dev_t = [t.to(ctx.dev) for t in draw_shared(B, N, SEED)]
    Q, R, S, Vr, Vs, dY = dev_t

    def step():
        Y, m, l = ctx.ck.sg_forward_raw(Q, R, S, Vr, Vs, None, w)
        ctx.ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w)
    ms = ctx.timed(step, steps, 3)
    ctx.ck.device_status()
    return {"workload": f"shared-KV B{B} Hq{HQ} N{N} w{w} per rank, independent replicas", "n_gpus": ctx.world,
            "scaling": "weak", "ms_per_step": ms, "value": ctx.world * 16 * D * triplets(B, HQ, N, w) / (ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "steps": steps}


def run_rows(args):
    ctx = Ctx(need_group=True)
    rec = rows_measure(ctx, args, args.steps)
    if ctx.rank == 0:
        rec.update(metric="fwd+bwd TFLOP/s, shared-KV causal w=128 d=128, row-sharded long sequence",
                   higher_is_better=True, dtype="bf16", data="synthetic")
        print(json.dumps(rec))
    ctx.close()


def run_replicas(args):
    ctx = Ctx(need_group=True)
    rec = replicas_measure(ctx, args, args.steps)
    if ctx.rank == 0:
        rec.update(metric=METRIC, higher_is_better=True, dtype="bf16", data="synthetic")
        print(json.dumps(rec))
    ctx.close()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--window", type=int, default=128, choices=[16, 32, 64, 128])
    ap.add_argument("--cpu-queries", type=int, default=4096)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--quick", action="store_true",
                    help="one GPU: only the headline problem (no window sweep, long sequence, secondary, reference kernels)")
    ap.add_argument("--seq-len", type=int, default=N, help="sequence length (profiling captures use a smaller case)")
    ap.add_argument("--batch", type=int, default=B)
    ap.add_argument("--heads", type=int, default=HQ, help="query heads (profiling a rank's share of the (batch, head) split)")
    ap.add_argument("--workload", default="auto", choices=["auto", "single", "scale", "batch", "rows", "heads", "other"],
                    help="auto: the headline problem on one GPU, or split by (batch, head) over N > 1 GPUs together with "
                         "the row-sharded long sequence and the replica run; batch: replicas only; rows: the row-sharded "
                         "long sequence only; other: the secondary configurations")
    ap.add_argument("--head-groups", type=int, default=0,
                    help="(batch, head) partition: ranks per batch shard (default: batches first)")
    ap.add_argument("--fwd-block", type=int, default=0, help="queries per forward CTA (0: built-in choice)")
    ap.add_argument("--bwd-block", type=int, default=0, help="queries per backward CTA (0: built-in choice)")
    ap.add_argument("--precise", action="store_true",
                    help="with --profile: time the compensated score products (value + residual split of Q o R)")
    ap.add_argument("--profile", action="store_true",
                    help="kernel-only run for profiler captures: exact warm-up count, no gate, no e2e and no CPU leg")
    ap.add_argument("--refgpu-child", action="store_true", help=argparse.SUPPRESS)
    a = ap.parse_args()
    N, B, HQ = a.seq_len, a.batch, a.heads
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if a.refgpu_child:
        refgpu_child(a)
    elif a.impl == "reference":
        run_reference(a)
    elif a.workload == "other":
        run_other(a)
    elif a.workload == "rows":
        run_rows(a)
    elif a.workload == "batch":
        run_replicas(a)
    elif a.workload in ("scale", "heads") or (a.workload == "auto" and world > 1):
        run_scale(a)
    else:
        run_single(a)
