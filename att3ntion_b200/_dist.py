"""Multi-GPU execution of the windowed single gather, one process per GPU.

Three partitionings, none of which puts a collective inside the kernels:

* batch / head sharding (``shard_batch``): independent problems, no communication.
* query-row sharding of one long sequence (``RowShardedGather``): rank r owns the
  contiguous rows [lo_r, hi_r) of Q, R, S, Vr, Vs.  A query sees the (window-1)
  keys before it, so before the forward each rank receives the last (window-1) key
  rows of its left neighbour (the halo; sent as one whole 128-row ring so that local
  and global ring slots coincide) into a local buffer, and after the backward
  it sends the key-gradient rows it produced for that halo back to the neighbour,
  which adds them to its own ("dK/dV reduced across ranks").  Both are point-to-point
  messages of (window-1) x D elements per tensor: latency-bound, one exchange per
  pass, no all-reduce.  Shard starts are multiples of 128 so every key keeps its ring
  slot and the sharded result is bit-identical to the single-GPU one for Y and dQ.

* head sharding of shared-KV problems (``HeadShardedGather``): the query heads of one KV head on
  different ranks; the key-side gradients are FP32 partials summed with one all-reduce per backward.

The reference has no multi-device path (its library never touches a communicator);
this module is new.  The compute step is injectable so the host logic (partitioning,
halo exchange, gradient hand-back) is testable with the ``gloo`` backend on CPU, where
the test-suite substitutes the CPU oracle for the kernels.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist

RING = 128


def shard_batch(n_items: int, world: int, rank: int) -> range:
    """Contiguous share of `n_items` independent (batch, head) problems for `rank`."""
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def row_shards(n: int, world: int, align: int = RING) -> list[tuple[int, int]]:
    """[lo, hi) query rows per rank: near-equal, every start a multiple of `align`
    (so ring slots coincide with the unsharded run); trailing ranks may be empty."""
    blocks = (n + align - 1) // align
    out, start = [], 0
    for r in range(world):
        take = blocks // world + (1 if r < blocks % world else 0)
        lo, hi = min(start * align, n), min((start + take) * align, n)
        out.append((lo, hi))
        start += take
    return out


@dataclass
class _Plan:
    lo: int
    hi: int
    halo: int          # key rows received from the left neighbour
    pad: int           # zero rows appended so the local length is a multiple of 16
    left: Optional[int]
    right: Optional[int]


class RowShardedGather:
    """Forward + backward of the windowed (shared- or independent-KV) single gather on
    row-sharded tensors.  ``compute_fwd(Q,R,S,Vr,Vs,window,q_begin) -> (Y,m,l)`` and
    ``compute_bwd(dY,Q,R,S,Vr,Vs,Y,m,l,window,q_begin) -> (dQ,dR,dS,dVr,dVs)`` default to the
    CUDA kernels."""

    def __init__(self, n_total: int, window: int, group=None,
                 compute_fwd: Optional[Callable] = None, compute_bwd: Optional[Callable] = None):
        if not 1 <= window <= RING:
            raise ValueError(f"window must be in [1,{RING}], got {window}")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.window = window
        self.shards = row_shards(n_total, self.world)
        lo, hi = self.shards[self.rank]
        active = [r for r, (a, b) in enumerate(self.shards) if b > a]
        pos = active.index(self.rank) if self.rank in active else -1
        # the halo is a whole ring (128 rows >= window - 1) so local key index = global index mod 128
        halo = min(RING, lo) if pos > 0 else 0
        n_local = halo + (hi - lo)
        self.plan = _Plan(lo, hi, halo, (-n_local) % 16,
                          active[pos - 1] if pos > 0 else None,
                          active[pos + 1] if 0 <= pos < len(active) - 1 else None)
        if compute_fwd is None or compute_bwd is None:
            from . import _cuda_kernels as ck
            compute_fwd = compute_fwd or (lambda Q, R, S, Vr, Vs, w, qb: ck.sg_forward_raw(Q, R, S, Vr, Vs, None, w, qb))
            compute_bwd = compute_bwd or (lambda dY, Q, R, S, Vr, Vs, Y, m, l, w, qb:
                                          ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w, qb))
        self._fwd, self._bwd = compute_fwd, compute_bwd
        self._saved = None

    # ------------------------------------------------------------------ communication
    def _global(self, r: int) -> int:
        return r if self.group is None else dist.get_global_rank(self.group, r)

    def _exchange(self, send: Optional[torch.Tensor], send_to: Optional[int],
                  recv: Optional[torch.Tensor], recv_from: Optional[int]) -> None:
        ops = []
        if send is not None and send_to is not None:
            ops.append(dist.P2POp(dist.isend, send, self._global(send_to), self.group))
        if recv is not None and recv_from is not None:
            ops.append(dist.P2POp(dist.irecv, recv, self._global(recv_from), self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()

    def _halo_rows_for_right(self) -> int:
        """Rows this rank sends to its right neighbour (that neighbour's halo length)."""
        if self.plan.right is None:
            return 0
        return min(RING, self.shards[self.plan.right][0])

    # ------------------------------------------------------------------ forward
    def forward(self, Q, R, S, Vr, Vs):
        """Local shards [B,H*,hi-lo,D] -> local Y [B,Hq,hi-lo,D] (and statistics kept for backward)."""
        p = self.plan
        if p.hi <= p.lo:
            self._saved = None
            return Q.new_zeros(Q.shape)
        kv = torch.stack([R, S, Vr, Vs])                              # [4,B,Hkv,n,D]
        n_send = self._halo_rows_for_right()
        send = kv[:, :, :, kv.size(3) - n_send:].contiguous() if n_send else None
        recv = kv.new_empty(4, *R.shape[:2], p.halo, R.shape[3]) if p.halo else None
        self._exchange(send, p.right, recv, p.left)
        if p.halo:
            kv = torch.cat([recv, kv], dim=3)
        pad = lambda t: torch.nn.functional.pad(t, (0, 0, 0, p.pad)) if p.pad else t
        Rl, Sl, Vrl, Vsl = (pad(kv[k]).contiguous() for k in range(4))
        Ql = torch.nn.functional.pad(Q, (0, 0, p.halo, p.pad)).contiguous()
        Y, m, l = self._fwd(Ql, Rl, Sl, Vrl, Vsl, self.window, p.halo)
        self._saved = (Ql, Rl, Sl, Vrl, Vsl, Y, m, l)
        return Y[:, :, p.halo:p.halo + (p.hi - p.lo)]

    # ------------------------------------------------------------------ backward
    def backward(self, dY):
        """Local cotangent [B,Hq,hi-lo,D] -> (dQ, dR, dS, dVr, dVs) for the local rows, with the
        contributions of the right neighbour's queries to this rank's last rows added in."""
        p = self.plan
        n_own = p.hi - p.lo
        if n_own <= 0 or self._saved is None:
            z = dY.new_zeros(dY.shape)
            return z, None, None, None, None
        Ql, Rl, Sl, Vrl, Vsl, Y, m, l = self._saved
        dYl = torch.nn.functional.pad(dY, (0, 0, p.halo, p.pad)).contiguous()
        dQ, dR, dS, dVr, dVs = self._bwd(dYl, Ql, Rl, Sl, Vrl, Vsl, Y, m, l, self.window, p.halo)
        dkv = torch.stack([dR, dS, dVr, dVs])                         # [4,B,Hkv,halo+n_own+pad,D]
        send = dkv[:, :, :, :p.halo].contiguous() if p.halo else None
        n_recv = self._halo_rows_for_right()
        recv = dkv.new_empty(4, *dR.shape[:2], n_recv, dR.shape[3]) if n_recv else None
        self._exchange(send, p.left, recv, p.right)
        own = dkv[:, :, :, p.halo:p.halo + n_own].clone()
        if n_recv:
            acc = torch.promote_types(own.dtype, torch.float32)       # BF16 partials are added in FP32
            own[:, :, :, n_own - n_recv:] = (own[:, :, :, n_own - n_recv:].to(acc) + recv.to(acc)).to(own.dtype)
        return (dQ[:, :, p.halo:p.halo + n_own], own[0], own[1], own[2], own[3])


class HeadShardedGather:
    """Shared-KV single gather with the query heads of each KV head split over the ranks of `group`
    (the second axis of the (batch, head) partition: batches go to different groups, the heads of one
    batch to the ranks of one group).  Rank r holds Q[:, heads_r] and dY[:, heads_r] and the whole key
    side R, S, Vr, Vs ([B,Hkv,N,D], the same on every rank of the group).

    The forward is local.  In the backward dQ is local, while every rank's key-side gradients are sums
    over its own heads only: the four FP32 partial tensors are stacked and summed over the group with
    one all-reduce (4 x [B,Hkv,N,D] floats) and rounded once afterwards -- the reduction the reference
    performs over its per-head partial buffers inside one GPU (cuda/backward.cu:2548-2575), done across
    GPUs.  ``compute_fwd(Q,R,S,Vr,Vs,window) -> (Y,m,l)`` and ``compute_bwd(dY,Q,R,S,Vr,Vs,Y,m,l,window)
    -> (dQ, dR, dS, dVr, dVs)`` with FP32 key gradients default to the CUDA kernels."""

    def __init__(self, window: int, group=None, compute_fwd: Optional[Callable] = None,
                 compute_bwd: Optional[Callable] = None):
        if not 1 <= window <= RING:
            raise ValueError(f"window must be in [1,{RING}], got {window}")
        self.group, self.window = group, window
        if compute_fwd is None or compute_bwd is None:
            from . import _cuda_kernels as ck
            compute_fwd = compute_fwd or (lambda Q, R, S, Vr, Vs, w: ck.sg_forward_raw(Q, R, S, Vr, Vs, None, w))
            compute_bwd = compute_bwd or (lambda dY, Q, R, S, Vr, Vs, Y, m, l, w:
                                          ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w, kv_f32=True))
        self._fwd, self._bwd = compute_fwd, compute_bwd
        self._saved = None

    @staticmethod
    def local_heads(hq: int, hkv: int, world: int, rank: int) -> list[int]:
        """Query heads of rank `rank`: the same share of every KV head's group of hq // hkv heads."""
        per_kv = hq // hkv
        if per_kv % world:
            raise ValueError(f"{per_kv} query heads per KV head do not split over {world} ranks")
        share = per_kv // world
        return [g * per_kv + rank * share + t for g in range(hkv) for t in range(share)]

    def forward(self, Q, R, S, Vr, Vs):
        Y, m, l = self._fwd(Q, R, S, Vr, Vs, self.window)
        self._saved = (Q, R, S, Vr, Vs, Y, m, l)
        return Y

    def backward(self, dY, out_dtype=None):
        """(dQ of the local heads, dR, dS, dVr, dVs summed over every rank's heads)."""
        Q, R, S, Vr, Vs, Y, m, l = self._saved
        dQ, dR, dS, dVr, dVs = self._bwd(dY, Q, R, S, Vr, Vs, Y, m, l, self.window)
        part = torch.stack([dR, dS, dVr, dVs]).to(torch.promote_types(dR.dtype, torch.float32))
        dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
        kv = part.to(out_dtype or R.dtype)
        return dQ, kv[0], kv[1], kv[2], kv[3]


def gather_rows(local: torch.Tensor, shards: Sequence[tuple[int, int]], group=None) -> torch.Tensor:
    """All-gathers row shards (dim 2) into the full tensor on every rank; for tests and checks."""
    world = dist.get_world_size(group)
    longest = max(hi - lo for lo, hi in shards)
    buf = torch.nn.functional.pad(local, (0, 0, 0, longest - local.size(2))).contiguous()
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf, group=group)
    return torch.cat([parts[r][:, :, :hi - lo] for r, (lo, hi) in enumerate(shards)], dim=2)
