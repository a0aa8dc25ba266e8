#!/usr/bin/env python
"""Benchmark of the shared-KV causal-window hot path (forward + all five gradients).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--window 128]

Workload (the shared-KV configuration the headline metric is quoted on): BF16, one
shared KV head, 8 query heads, D = 128, batch 4, N = 8192, causal window 128;
Q/R/S/Vr/Vs ~ N(0,1)/sqrt(128) from seed 3, dY ~ N(0,1).  A step is one forward
plus one backward over that batch.  With N GPUs every rank runs its own batch of
the same shape (weak scaling over the data-parallel batch axis, no collective on
the data path); the value is the job's total algorithmic TFLOP/s.

Algorithmic FLOPs per step = 16 * D * T with T = B * Hq * sum_i min(i+1, w)^2
(forward 4*D*T: score and value contraction; backward 12*D*T: six contractions).

One JSON line is printed by rank 0.  `value` is device time with inputs resident;
`e2e` times the public API call with pinned host buffers, host<->device copies
included.  `--impl reference` times the CPU restatement of the reference's naive
path (oracle/triplet_oracle.py) on the host cores instead.
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
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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


def draw_inputs(window):
    g = torch.Generator(device="cpu").manual_seed(SEED)
    s = 1.0 / math.sqrt(D)
    Q = (torch.randn(B, HQ, N, D, generator=g) * s).to(torch.bfloat16)
    kv = [(torch.randn(B, HKV, N, D, generator=g) * s).to(torch.bfloat16) for _ in range(4)]
    dY = torch.randn(B, HQ, N, D, generator=g).to(torch.bfloat16)
    return Q, kv, dY


# --------------------------------------------------------------------------- CPU arm (oracle port)

def cpu_sample(window, queries=4096, batch=1):
    """fwd+bwd of the banded FP32 restatement on `queries` interior queries of one
    batch (all 8 heads, full window) with every host thread.  Returns (TFLOP/s, seconds, cores)."""
    from oracle import triplet_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = queries + window - 1
    n += (-n) % 16
    g = torch.Generator(device="cpu").manual_seed(SEED)
    s = 1.0 / math.sqrt(D)
    Q = (torch.randn(batch, HQ, n, D, generator=g) * s).to(torch.bfloat16)
    kv = [(torch.randn(batch, HKV, n, D, generator=g) * s).to(torch.bfloat16) for _ in range(4)]
    dY = torch.randn(batch, HQ, n, D, generator=g).to(torch.bfloat16)
    q_begin = n - queries
    t0 = time.perf_counter()
    O.single_gather_banded(Q, *kv, window=window, dY=dY, chunk=32, q_begin=q_begin, dtype=torch.float32)
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
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"shared-KV B{B} Hq{HQ} Hkv{HKV} N{N} D{D} causal window {args.window}",
                   "note": "each step is a bounded sample of that workload on the host cores"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# --------------------------------------------------------------------------- GPU arm

def run_ours(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the sm_100a kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from att3ntion_b200 import _cabi, _cuda_kernels as ck, single_gather_shared_attention
    lib = _cabi.lib
    w = args.window
    Qh, kvh, dYh = draw_inputs(w)
    host_in = [t.pin_memory() for t in (Qh, *kvh, dYh)]
    Q, R, S, Vr, Vs, dY = (t.to(dev, non_blocking=True) for t in host_in)
    torch.cuda.synchronize()
    flops_step = 16 * D * triplets(B, HQ, N, w)

    def step():
        Y, m, l = ck.sg_forward_raw(Q, R, S, Vr, Vs, None, w)
        return Y, ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.__enter__()                      # nvidia-smi needs a moment to start: begin before the warm-up
    for _ in range(args.warmup if args.profile else max(args.warmup, 3)):
        step()
    barrier()
    lib.att3_timing_enable(1)
    for k in range(6):
        tot, cnt = C.c_double(), C.c_ulonglong()
        lib.att3_timing_read(k, C.byref(tot), C.byref(cnt))          # drop anything recorded during warm-up
    launches0 = [lib.att3_launch_count(i) for i in range(4)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    sampler.__exit__()
    clocks = sampler
    ms = e0.elapsed_time(e1)
    launches = sum(lib.att3_launch_count(i) for i in range(4)) - sum(launches0)
    ktime = {}
    for k, name in enumerate(["sg_ring_fwd", "sg_ring_bwd", "sg_bwd_reduce"]):
        tot, cnt = C.c_double(), C.c_ulonglong()
        lib.att3_timing_read(k, C.byref(tot), C.byref(cnt))
        ktime[name] = (tot.value, cnt.value)
    lib.att3_timing_enable(0)
    ck.device_status()
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    ms_step = ms / args.steps
    value = world * flops_step / (ms_step * 1e-3) / 1e12

    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "ms_per_step": ms_step, "value": value,
                              "kernel_ms": {k: (v[0] / v[1] if v[1] else None) for k, v in ktime.items()}}))
        return

    # --- end to end through the public API with host buffers (pinned), copies inside the timed region
    host_out = [torch.empty_like(t).pin_memory() for t in (Qh, Qh, *kvh)]     # Y, dQ, dR, dS, dVr, dVs
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    # Every step copies its own inputs host -> device and its own results device -> host; the copies run on
    # two side streams, so the input copy of step k+1 and the result copy of step k-1 overlap the kernels of
    # step k (double-buffered device inputs), as an input pipeline in front of a training step would.
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

    def e2e_step(k):
        slot = k & 1
        main.wait_event(in_ready[slot])
        q, r, s, vr, vs, dy = dev_in[slot]
        leaves = [t.detach().requires_grad_(True) for t in (q, r, s, vr, vs)]
        y = single_gather_shared_attention(*leaves, None, window=w)
        y.backward(dy)
        consumed[slot].record(main)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            host_out[0].copy_(y.detach(), non_blocking=True)
            y.record_stream(s_out)
            for dst, leaf in zip(host_out[1:], leaves):
                dst.copy_(leaf.grad, non_blocking=True)
                leaf.grad.record_stream(s_out)
        keep[slot] = (y, leaves)

    def e2e_run(steps):
        prefetch(0)
        for k in range(steps):
            if k + 1 < steps:
                prefetch(k + 1)
            e2e_step(k)
        main.wait_stream(s_out)                          # the last results are on the host when the clock stops

    e2e_steps = max(2, min(args.steps, 20))
    e2e_run(2)
    barrier()
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = t.item()
    e2e_value = world * flops_step / (e2e_ms / e2e_steps * 1e-3) / 1e12

    if rank == 0:
        burst, sustained, src = measured_peaks()
        bwd_ms, bwd_n = ktime["sg_ring_bwd"]
        # dominant kernel: one backward pass launch produces one key side's gradients (and dQ once),
        # half of the backward's 12*D*T algorithmic FLOPs
        flops_launch = 6 * D * triplets(B, HQ, N, w)
        achieved = flops_launch / (bwd_ms / max(1, bwd_n) * 1e-3) / 1e12 if bwd_n else None
        roofline = {"bound": "tensor", "kernel": "sg_ring_bwd_kernel<128>", "achieved": achieved, "peak": sustained,
                    "unit": "TFLOP/s", "frac": (achieved / sustained) if achieved else None,
                    "peak_source": f"{src} bf16_tflops_sustained (kernel timed inside the step loop)",
                    "frac_of_burst_peak": (achieved / burst) if achieved else None,
                    "traffic": traffic_bytes_per_launch(B, HQ, HKV, N, D, w),
                    "kernel_ms": {k: (v[0] / v[1] if v[1] else None) for k, v in ktime.items()},
                    "step_frac_of_sustained_peak": value / world / sustained}
        cpu_v, cpu_dt, cores = cpu_sample(w, queries=args.cpu_queries) if world == 1 and not args.no_cpu else (None, 0, 0)
        out = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"shared-KV B{B} Hq{HQ} Hkv{HKV} N{N} D{D} causal window {w}, fwd + 5 gradients",
                       "per_gpu_batch": B, "parallelism": f"dp{world} over batch, no data-path collective",
                       "l2": "inputs+outputs 0.5 GB per step exceed the 126 MB L2; no explicit flush",
                       "flops_per_step": flops_step},
            "clocks": clocks.summary(),
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps,
                    "copies": "every step's inputs and results cross PCIe inside the timed region, on two side "
                              "streams that overlap the neighbouring steps' kernels"},
            "gpu_launches": int(launches),
            "roofline": roofline,
        }
        if cpu_v is not None:
            out["cpu_baseline"] = {"value": cpu_v, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                   "sample": f"banded FP32 torch restatement of the naive path, 1 batch x 8 heads x "
                                             f"{args.cpu_queries} interior queries, {cpu_dt:.1f} s"}
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def run_rows(args):
    """Long-sequence workload: B1 Hq8 Hkv1 N131072 D128 w128, query rows
    sharded over the ranks with a 128-row key halo from the left neighbour and the halo key
    gradients handed back after the backward (two point-to-point messages per step, NCCL).
    Total work is fixed, so the scaling is strong."""
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from att3ntion_b200 import _cabi, _cuda_kernels as ck
    from att3ntion_b200._dist import RowShardedGather
    n, w = args.seq_len if args.seq_len != 8192 else 131072, args.window
    op = RowShardedGather(n, w)
    lo, hi = op.plan.lo, op.plan.hi
    g = torch.Generator(device="cpu").manual_seed(4)
    s = 1.0 / math.sqrt(D)
    # every rank draws the full tensors from the same seed and keeps its rows (inputs are row-sharded)
    def draw(heads, scale):
        return (torch.randn(1, heads, n, D, generator=g) * scale).to(torch.bfloat16)[:, :, lo:hi].contiguous().to(dev)
    Q = draw(HQ, s); R = draw(1, s); S = draw(1, s); Vr = draw(1, s); Vs = draw(1, s); dY = draw(HQ, 1.0)
    flops_step = 16 * D * triplets(1, HQ, n, w)

    def step():
        y = op.forward(Q, R, S, Vr, Vs)
        return y, op.backward(dY)

    for _ in range(max(args.warmup, 3)):
        step()
    dist.barrier(); torch.cuda.synchronize()
    l0 = sum(_cabi.lib.att3_launch_count(i) for i in range(4))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = step()
    e1.record()
    dist.barrier(); torch.cuda.synchronize()
    ck.device_status()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    launches = sum(_cabi.lib.att3_launch_count(i) for i in range(4)) - l0
    chk = torch.stack([out[0].float().abs().mean(), out[1][0].float().abs().mean(), out[1][1].float().abs().mean()])
    dist.all_reduce(chk)
    if rank == 0:
        print(json.dumps({
            "metric": "fwd+bwd TFLOP/s, shared-KV causal w=128 d=128, row-sharded long sequence",
            "value": flops_step / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"shared-KV B1 Hq{HQ} Hkv1 N{n} D{D} causal window {w}, rows sharded over "
                                   f"{world} GPU(s), 128-row key halo, halo key-gradients handed back",
                       "shards": op.shards, "flops_per_step": flops_step},
            "gpu_launches": int(launches), "checksum": [round(v, 6) for v in chk.tolist()],
        }))
    dist.destroy_process_group()


def run_heads(args):
    """Config 4 itself (B4 Hq8 Hkv1 N8192 D128) partitioned over the ranks by (batch, head): the batches are
    split over batch shards and the query heads of a batch shard over the ranks of its group, whose FP32
    key-gradient partials are summed with one NCCL all-reduce per step (4 x [b,1,N,128] floats).  Total work is
    fixed, so the scaling is strong.  --head-groups sets the ranks per batch shard."""
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from att3ntion_b200 import _cabi, _cuda_kernels as ck
    from att3ntion_b200._dist import HeadShardedGather, shard_batch
    n, w, Bt = args.seq_len, args.window, args.batch
    # Default factorisation: keep two batches per rank as long as the heads can take the rest.  A backward block is
    # at least 128 queries, so one 8192-row sequence per rank gives 64 CTAs for 148 SMs, two give 128: per-rank
    # step times on one GPU are 7.07 ms for B1 Hq8 against 4.34 ms for B2 Hq4, 3.78 ms for B1 Hq4 against 2.44 ms
    # for B2 Hq2.
    hg = args.head_groups
    if not hg:
        bs = max(d for d in range(1, world + 1) if world % d == 0 and d <= max(1, Bt // 2))
        hg = world // bs
        if HQ % hg:
            hg = max(1, world // min(world, Bt))
    if world % hg or HQ % hg:
        raise SystemExit(f"bench.py: {world} ranks do not split into head groups of {hg}")
    bshards = world // hg
    brank, hrank = rank // hg, rank % hg
    groups = [dist.new_group(list(range(b * hg, (b + 1) * hg))) for b in range(bshards)]
    op = HeadShardedGather(w, group=groups[brank])
    batches = list(shard_batch(Bt, bshards, brank))
    heads = HeadShardedGather.local_heads(HQ, 1, hg, hrank)
    g = torch.Generator(device="cpu").manual_seed(3)
    s = 1.0 / math.sqrt(D)
    def draw(nh, scale, hsel=None):
        t = (torch.randn(Bt, nh, n, D, generator=g) * scale).to(torch.bfloat16)[batches]
        return (t[:, hsel] if hsel is not None else t).contiguous().to(dev)
    Q = draw(HQ, s, heads); R = draw(1, s); S = draw(1, s); Vr = draw(1, s); Vs = draw(1, s); dY = draw(HQ, 1.0, heads)
    flops_step = 16 * D * triplets(Bt, HQ, n, w)

    def step():
        if not batches:
            return None
        y = op.forward(Q, R, S, Vr, Vs)
        return y, op.backward(dY)

    for _ in range(max(args.warmup, 3)):
        step()
    dist.barrier(); torch.cuda.synchronize()
    l0 = sum(_cabi.lib.att3_launch_count(i) for i in range(4))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = step()
    e1.record()
    dist.barrier(); torch.cuda.synchronize()
    ck.device_status()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    launches = sum(_cabi.lib.att3_launch_count(i) for i in range(4)) - l0
    chk = torch.zeros(3, device=dev)
    if out is not None:
        # Y and dQ summed over everything; the key gradient counted once per batch shard (head rank 0)
        chk = torch.stack([out[0].float().abs().sum(), out[1][0].float().abs().sum(),
                           out[1][1].float().abs().sum() * (1.0 if hrank == 0 else 0.0)])
    dist.all_reduce(chk)
    if rank == 0:
        print(json.dumps({
            "metric": "fwd+bwd TFLOP/s, shared-KV causal w=128 d=128, (batch, head) partition",
            "value": flops_step / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"shared-KV B{Bt} Hq{HQ} Hkv1 N{n} D{D} causal window {w}, {bshards} batch shard(s) x "
                                   f"{hg} head group(s); key-gradient partials all-reduced inside a batch shard",
                       "allreduce_bytes_per_step": (4 * len(batches) * n * D * 4) if hg > 1 else 0,
                       "flops_per_step": flops_step},
            "gpu_launches": int(launches), "checksum": [round(v, 3) for v in chk.tolist()],
        }))
    dist.destroy_process_group()


def run_other(args):
    """Secondary configurations, one GPU, device-resident inputs, CUDA events, median of `--steps`
    repeats: C3 = independent-head single gather B4 H8 N2048 D64 w128 (16*D*T FLOPs), C2 = three-gather
    operator B8 H4 N256 D64 without mask or scatter (3*(4+14)*D*B*H*N^3 FLOPs, the reference's own count), and
    the same shape with the scatter outputs switched on (time only)."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the sm_100a kernels have no CPU path")
    from att3ntion_b200 import _cuda_kernels as ck
    dev = torch.device("cuda", 0)
    reps = max(3, min(args.steps, 20))

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    out = {}
    g = torch.Generator(device="cpu").manual_seed(2)
    b3, h3, n3, d3, w3 = 4, 8, 2048, 64, 128
    t5 = [(torch.randn(b3, h3, n3, d3, generator=g) / math.sqrt(d3)).to(torch.bfloat16).to(dev) for _ in range(5)]
    dy = torch.randn(b3, h3, n3, d3, generator=g).to(torch.bfloat16).to(dev)

    def c3():
        Y, m, l = ck.sg_forward_raw(*t5, None, w3)
        ck.sg_backward_raw(dy, *t5, Y, m, l, None, w3)
    ms = timed(c3)
    fl = 16 * d3 * triplets(b3, h3, n3, w3)
    out["C3 single gather B4 H8 N2048 D64 w128"] = {"ms": ms, "TFLOP/s": fl / ms / 1e9}

    g = torch.Generator(device="cpu").manual_seed(1)
    b2, h2, n2, d2 = 8, 4, 256, 64
    ins = [(torch.randn(b2, h2, n2, d2, generator=g) * (0.5 if k < 3 else 1.0)).to(torch.bfloat16).to(dev) for k in range(9)]
    for k in (4, 6, 8):
        ins[k].zero_()
    cot = [torch.randn(b2, h2, n2, d2, generator=g).to(torch.bfloat16).to(dev) for _ in range(3)] + \
          [torch.zeros(b2, h2, n2, d2, dtype=torch.bfloat16, device=dev) for _ in range(3)]

    def c2():
        o = ck.forward(*ins, 0.0, -1, -1, -1, None, 0)
        ck.backward(*cot, *ins, *o[6:12], 0.0, None, o[0], o[1], o[2])
    ms = timed(c2)
    fl = 3 * (4 + 14) * d2 * b2 * h2 * n2 ** 3
    out["C2 three-gather B8 H4 N256 D64"] = {"ms": ms, "TFLOP/s": fl / ms / 1e9}

    # The same shape with the second value tensors in use (module option scatter=True): three scatter outputs
    # and their cross terms in all nine gradients, on CUDA cores.  No FLOP model is published for this part,
    # so only the time is reported.
    ins2 = [t.clone() for t in ins]
    for k in (4, 6, 8):
        ins2[k] = torch.randn(b2, h2, n2, d2, generator=g).to(torch.bfloat16).to(dev)
    cot2 = cot[:3] + [torch.randn(b2, h2, n2, d2, generator=g).to(torch.bfloat16).to(dev) for _ in range(3)]

    def c2s():
        o = ck.forward(*ins2, 0.0, -1, -1, -1, None, 0)
        ck.backward(*cot2, *ins2, *o[6:12], 0.0, None, o[0], o[1], o[2])
    ms = timed(c2s)
    out["C2 with scatter outputs (second value tensors non-zero)"] = {"ms": ms}
    ck.device_status()
    print(json.dumps({"secondary_configs": out, "repeats": reps, "data": "synthetic"}))


# DRAM bytes (read + write) of one sg_ring_bwd_kernel launch, from the ncu capture summarised in
# profiles/sg_ring_w128_d128_pipelined.md: 162.5 MB (key side S + dQ) and 140.0 MB (key side R) at
# B4 Hq8 Hkv1 N4096 D128 w128, i.e. 9232 bytes per (batch, query) on average over the two launches
# of a step.  The traffic is per-row streaming (Q, dY, Y rows, key rows, FP32 partial rows), so it
# scales with B*N; other head counts, head sizes or windows have not been captured (None).
def traffic_bytes_per_launch(B, Hq, Hkv, N, D, w):
    if (Hq, Hkv, D, w) == (8, 1, 128, 128):
        return 9232 * B * N
    return None


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--window", type=int, default=128, choices=[16, 32, 64, 128])
    ap.add_argument("--cpu-queries", type=int, default=4096)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--seq-len", type=int, default=N, help="sequence length (profiling captures use a smaller case)")
    ap.add_argument("--batch", type=int, default=B)
    ap.add_argument("--workload", default="batch", choices=["batch", "rows", "heads", "other"],
                    help="batch: config 4, one batch per GPU (default); rows: config 5, one sequence row-sharded; "
                         "heads: config 4 split by (batch, head) with the key-gradient all-reduce (strong scaling)")
    ap.add_argument("--head-groups", type=int, default=0,
                    help="heads workload: ranks per batch shard (default: as few as keep two batches per rank)")
    ap.add_argument("--profile", action="store_true",
                    help="kernel-only run for profiler captures: exact warm-up count, no e2e and no CPU leg")
    a = ap.parse_args()
    N, B = a.seq_len, a.batch
    if a.impl == "reference":
        run_reference(a)
    elif a.workload == "other":
        run_other(a)
    elif a.workload == "rows":
        run_rows(a)
    elif a.workload == "heads":
        run_heads(a)
    else:
        run_ours(a)
