"""Worker of tests/test_dist_gpu.py: one process per GPU (torch.distributed.run), NCCL.  Runs the row-sharded and
the head-sharded operators of att3ntion_b200._dist with the real kernels and compares every rank's results with
the same problem computed whole on that rank's own GPU."""
import math
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))


def draw(B, Hq, N, D, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    s = 1.0 / math.sqrt(D)
    Q = (torch.randn(B, Hq, N, D, generator=g) * s).to(torch.bfloat16)
    kv = [(torch.randn(B, 1, N, D, generator=g) * s).to(torch.bfloat16) for _ in range(4)]
    dY = torch.randn(B, Hq, N, D, generator=g).to(torch.bfloat16)
    return Q, kv, dY


def close(a, b, rel_tol, what):
    a, b = a.float(), b.float()
    rel = ((a - b).norm() / b.norm().clamp_min(1e-12)).item()
    assert rel <= rel_tol, f"{what}: rel-L2 {rel}"


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    from att3ntion_b200 import _cuda_kernels as ck
    from att3ntion_b200._dist import HeadShardedGather, RowShardedGather

    # ---- rows: one sequence of 128 * 6 * world rows, window 128 (ring schedule) and 32 (packed schedule)
    for w in (128, 32):
        B, Hq, N, D = 1, 8, 768 * world, 128
        Q, kv, dY = draw(B, Hq, N, D, seed=4 + w)
        full = [t.to(dev) for t in (Q, *kv)]
        Y, m, l = ck.sg_forward_raw(*full, None, w)
        G = ck.sg_backward_raw(dY.to(dev), *full, Y, m, l, None, w)
        op = RowShardedGather(N, w)
        lo, hi = op.plan.lo, op.plan.hi
        Ys = op.forward(*[t[:, :, lo:hi].contiguous() for t in full])
        gs = op.backward(dY.to(dev)[:, :, lo:hi].contiguous())
        ck.device_status()
        assert torch.equal(Ys, Y[:, :, lo:hi]), f"rows w{w}: Y differs on rank {rank}"
        assert torch.equal(gs[0], G[0][:, :, lo:hi]), f"rows w{w}: dQ differs on rank {rank}"
        for k in range(1, 5):
            close(gs[k], G[k][:, :, lo:hi], 4e-3, f"rows w{w}: key gradient {k} on rank {rank}")

    # ---- heads: the query heads of each KV head split over the ranks, key gradients all-reduced per key side
    for w in (128, 16):
        B, Hq, N, D = 2, 8 * world, 512, 128
        Q, kv, dY = draw(B, Hq, N, D, seed=9 + w)
        full = [t.to(dev) for t in (Q, *kv)]
        Y, m, l = ck.sg_forward_raw(*full, None, w)
        G = ck.sg_backward_raw(dY.to(dev), *full, Y, m, l, None, w)
        heads = HeadShardedGather.local_heads(Hq, 1, world, rank)
        op = HeadShardedGather(w)
        Ys = op.forward(full[0][:, heads].contiguous(), *full[1:])
        gs = op.backward(dY.to(dev)[:, heads].contiguous())
        ck.device_status()
        assert torch.equal(Ys, Y[:, heads]), f"heads w{w}: Y differs on rank {rank}"
        assert torch.equal(gs[0], G[0][:, heads]), f"heads w{w}: dQ differs on rank {rank}"
        for k in range(1, 5):
            close(gs[k], G[k], 4e-3, f"heads w{w}: key gradient {k} on rank {rank}")
    dist.barrier()
    if rank == 0:
        print("dist-gpu-ok", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
