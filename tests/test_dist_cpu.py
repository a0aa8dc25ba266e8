"""World-size-2 (and 3) gloo runs of the multi-GPU host logic on CPU: partitioning,
halo exchange, the hand-back of halo key gradients, the per-side all-reduce of the head
partition and what a rank sees when its neighbour fails before an exchange.  The compute
step is the CPU oracle here (the kernels need a GPU); what is under test is
att3ntion_b200/_dist.py."""
import datetime
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import triplet_oracle as O

NAMES = ["Q", "R", "S", "Vr", "Vs"]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_fwd(Q, R, S, Vr, Vs, w, qb):
    r = O.single_gather_banded(Q, R, S, Vr, Vs, window=w, q_begin=qb, chunk=32)
    return r["Y"], r["m"], r["l"]


def _oracle_bwd(dY, Q, R, S, Vr, Vs, Y, m, l, w, qb):
    r = O.single_gather_banded(Q, R, S, Vr, Vs, window=w, dY=dY, q_begin=qb, chunk=32)
    return r["dQ"], r["dR"], r["dS"], r["dVr"], r["dVs"]


def _worker(rank, world, port, n, window, hkv, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from att3ntion_b200._dist import RowShardedGather, gather_rows
        g = torch.Generator().manual_seed(4)
        full = {"Q": torch.randn(1, 4, n, 16, generator=g, dtype=torch.float64)}
        for k in NAMES[1:]:
            full[k] = torch.randn(1, hkv, n, 16, generator=g, dtype=torch.float64)
        dY = torch.randn(1, 4, n, 16, generator=g, dtype=torch.float64)
        op = RowShardedGather(n, window, compute_fwd=_oracle_fwd, compute_bwd=_oracle_bwd)
        lo, hi = op.plan.lo, op.plan.hi
        Y = op.forward(*[full[k][:, :, lo:hi].contiguous() for k in NAMES])
        grads = op.backward(dY[:, :, lo:hi].contiguous())
        got = [gather_rows(Y, op.shards)] + [gather_rows(t, op.shards) for t in grads]
        if rank == 0:
            ref = O.single_gather_banded(*[full[k] for k in NAMES], window=window, dY=dY, chunk=32)
            errs = [(a - ref[k]).abs().max().item() for a, k in zip(got, ["Y", "dQ", "dR", "dS", "dVr", "dVs"])]
            torch.save({"errs": errs, "shards": op.shards}, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,window,hkv", [(2, 400, 128, 1), (2, 272, 33, 4), (3, 300, 64, 1)])
def test_row_sharding_matches_unsharded(tmp_path, world, n, window, hkv):
    out = str(tmp_path / "res.pt")
    mp.spawn(_worker, args=(world, _free_port(), n, window, hkv, out), nprocs=world, join=True)
    res = torch.load(out)
    assert max(res["errs"]) < 1e-9, res
    assert res["shards"][0][0] == 0 and res["shards"][-1][1] == n
    assert all(lo % 128 == 0 for lo, _ in res["shards"])


def _head_worker(rank, world, port, hkv, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from att3ntion_b200._dist import HeadShardedGather
        n, window, hq = 160, 48, 4 * hkv
        g = torch.Generator().manual_seed(9)
        full = {"Q": torch.randn(2, hq, n, 16, generator=g, dtype=torch.float64)}
        for k in NAMES[1:]:
            full[k] = torch.randn(2, hkv, n, 16, generator=g, dtype=torch.float64)
        dY = torch.randn(2, hq, n, 16, generator=g, dtype=torch.float64)
        fwd = lambda Q, R, S, Vr, Vs, w: _oracle_fwd(Q, R, S, Vr, Vs, w, 0)
        def bwd(dY_, Q, R, S, Vr, Vs, Y, m, l, w, between):
            dQ, dR, dS, dVr, dVs = _oracle_bwd(dY_, Q, R, S, Vr, Vs, Y, m, l, w, 0)
            kv = torch.stack([dS, dVs, dR, dVr])
            between(kv[:2])                      # the first key side is summed while the second is "computed"
            return dQ, kv
        op = HeadShardedGather(window, compute_fwd=fwd, compute_bwd=bwd)
        heads = HeadShardedGather.local_heads(hq, hkv, world, rank)
        Y = op.forward(full["Q"][:, heads].contiguous(), *[full[k] for k in NAMES[1:]])
        dQ, dR, dS, dVr, dVs = op.backward(dY[:, heads].contiguous())
        ref = O.single_gather_banded(*[full[k] for k in NAMES], window=window, dY=dY, chunk=32)
        errs = [(Y - ref["Y"][:, heads]).abs().max().item(), (dQ - ref["dQ"][:, heads]).abs().max().item()]
        errs += [(a - ref[k]).abs().max().item() for a, k in zip((dR, dS, dVr, dVs), ["dR", "dS", "dVr", "dVs"])]
        torch.save({"errs": errs, "heads": heads}, f"{out}.{rank}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("hkv", [1, 2])
def test_head_sharding_sums_key_gradients_over_ranks(tmp_path, hkv):
    """Two ranks, each with half of the query heads of every KV head: Y and dQ are the local slices of
    the unsharded result, the key gradients on every rank are the full sums."""
    out = str(tmp_path / "res.pt")
    mp.spawn(_head_worker, args=(2, _free_port(), hkv, out), nprocs=2, join=True)
    seen = []
    for rank in range(2):
        res = torch.load(f"{out}.{rank}")
        assert max(res["errs"]) < 1e-9, res
        seen += res["heads"]
    assert sorted(seen) == list(range(4 * hkv))


def _failing_worker(rank, world, port, mode, out):
    """Rank 1 fails before the halo exchange of the forward.  mode "store": it records the failure on the
    store first (guard), so rank 0 stops at its host-side check; mode "silent": it just never joins, so
    rank 0's exchange runs into the process group's timeout.  Either way rank 0 must get PeerExchangeError
    instead of blocking."""
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=20))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=4))
    from att3ntion_b200 import _dist
    n, window = 400, 64
    g = torch.Generator().manual_seed(1)
    full = [torch.randn(1, 2, n, 16, generator=g, dtype=torch.float64)] + \
           [torch.randn(1, 1, n, 16, generator=g, dtype=torch.float64) for _ in range(4)]
    op = _dist.RowShardedGather(n, window, compute_fwd=_oracle_fwd, compute_bwd=_oracle_bwd, store=store)
    lo, hi = op.plan.lo, op.plan.hi
    t0 = time.monotonic()
    result = "completed"
    try:
        with _dist.guard(store, rank):
            if rank == 1:
                if mode == "store":
                    raise ValueError("injected failure before the halo exchange")
                time.sleep(8)                     # silent: outlives the peer's timeout without joining
                result = "slept"
            else:
                if mode == "store":
                    time.sleep(1.0)               # let the failure note land first
                op.forward(*[t[:, :, lo:hi].contiguous() for t in full])
    except _dist.PeerExchangeError as e:
        result = f"peer-error: {e}"
    except ValueError as e:
        result = f"raised: {e}"
    torch.save({"result": result, "seconds": time.monotonic() - t0}, f"{out}.{rank}")
    # no destroy_process_group: a rank whose peer is gone must not wait for it at shutdown either
    os._exit(0)


@pytest.mark.parametrize("mode", ["store", "silent"])
def test_neighbour_failure_is_reported_not_waited_for(tmp_path, mode):
    out = str(tmp_path / "res.pt")
    mp.spawn(_failing_worker, args=(2, _free_port(), mode, out), nprocs=2, join=True)
    r0, r1 = torch.load(f"{out}.0"), torch.load(f"{out}.1")
    assert r0["result"].startswith("peer-error"), r0
    assert r0["seconds"] < 7.5, r0                                 # bounded by the 4 s group timeout, not by the peer
    if mode == "store":
        assert "injected failure" in r0["result"] and r1["result"].startswith("raised"), (r0, r1)
        assert r0["seconds"] < 3.0, r0                             # learnt on the host, no exchange attempted


def test_partition_helpers():
    from att3ntion_b200._dist import row_shards, shard_batch
    assert row_shards(131072, 8) == [(i * 16384, (i + 1) * 16384) for i in range(8)]
    s = row_shards(300, 4)
    assert s[0] == (0, 128) and s[-1][1] == 300 and sum(hi - lo for lo, hi in s) == 300
    assert [len(shard_batch(10, 4, r)) for r in range(4)] == [3, 3, 2, 2]
    assert list(shard_batch(4, 8, 5)) == []
