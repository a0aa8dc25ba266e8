"""Multi-GPU execution of the windowed single gather, one process per GPU.

Three partitionings, none of which puts a collective inside the kernels:

* batch / head sharding (``shard_batch``): independent problems, no communication.
* query-row sharding of one long sequence (``RowShardedGather``): rank r owns the
  contiguous rows [lo_r, hi_r) of Q, R, S, Vr, Vs.  A query sees the (window-1)
  keys before it, so before the forward each rank receives the last key rows of its
  left neighbour (the halo; one whole 128-row ring so that local and global ring
  slots coincide) straight into the front of its local key buffers, and after the
  backward it sends the FP32 key-gradient rows it produced for that halo back to
  the neighbour, which adds them to its own in FP32 and rounds once ("dK/dV reduced
  across ranks").  Both are point-to-point messages of 128 x D elements per tensor:
  latency-bound, one exchange per pass, no all-reduce.  Shard starts are multiples
  of 128 so every key keeps its ring slot: Y and dQ are bit-identical to the
  single-GPU run, and so are the key gradients except on the 127 rows before a shard
  boundary, where the same FP32 terms are added in another order before the one
  rounding.
* head sharding of shared-KV problems (``HeadShardedGather``): the query heads of one
  KV head on different ranks; the key-side gradients are FP32 partials summed with
  one all-reduce per key side, the first of which is issued while the second side
  is still being computed.

The reference has no multi-device path (its library never touches a communicator);
this module is new.  The compute step is injectable so the host logic (partitioning,
halo exchange, gradient hand-back, failure reporting) is testable with the ``gloo``
backend on CPU, where the test-suite substitutes the CPU oracle for the kernels.

Failure handling.  Every exchange is bounded by the process group's timeout: a
neighbour that never posts its half (it raised, exited or hangs before the exchange)
makes ``wait`` fail, and the failure surfaces as ``PeerExchangeError`` instead of a
rank blocked forever.  A rank that fails *before* an exchange can call
``notify_failure`` (or use ``guard``) so that its peers learn of it through the
store ahead of their next launch and stop without waiting for the timeout.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist

RING = 128


class PeerExchangeError(RuntimeError):
    """A halo exchange, gradient hand-back or all-reduce did not complete (a peer failed or timed out)."""


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


# --------------------------------------------------------------------------- failure notes on the store

_FAIL_KEY = "att3_dist_failed"


def notify_failure(store, rank: int, what: str) -> None:
    """Records on the rendezvous store that `rank` has failed; peers see it in `check_peers`."""
    store.set(_FAIL_KEY, f"rank {rank}: {what}")


def check_peers(store) -> None:
    """Raises PeerExchangeError if any rank has recorded a failure.  Host-side and cheap: meant to be
    called between steps, before the next launch, so nobody enters an exchange a dead peer will never join."""
    if store is None:
        return
    if store.check([_FAIL_KEY]):
        raise PeerExchangeError(f"a peer reported a failure: {store.get(_FAIL_KEY).decode()}")


@contextlib.contextmanager
def guard(store, rank: int):
    """Runs a step; an exception inside is recorded on the store for the peers before it propagates."""
    try:
        yield
    except PeerExchangeError:
        raise
    except BaseException as e:          # noqa: BLE001 -- recorded and re-raised
        if store is not None:
            notify_failure(store, rank, f"{type(e).__name__}: {e}")
        raise


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
    CUDA kernels (key gradients left in FP32 until the halo contributions are in).

    The local key tensors live in one buffer [4,B,Hkv,halo+n+pad,D] that is allocated once; the halo
    is received into its front rows and the shard's own rows are copied in behind it (or, through
    ``local_buffers``, written there by the caller in the first place), so a forward makes no
    ``cat``/``stack`` copies."""

    def __init__(self, n_total: int, window: int, group=None,
                 compute_fwd: Optional[Callable] = None, compute_bwd: Optional[Callable] = None, store=None):
        if not 1 <= window <= RING:
            raise ValueError(f"window must be in [1,{RING}], got {window}")
        self.group = group
        self.store = store
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
                                          ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w, qb, kv_f32=True))
        self._fwd, self._bwd = compute_fwd, compute_bwd
        self._saved = None
        self._kv = self._q = self._dy = None       # local buffers, allocated at first use

    # ------------------------------------------------------------------ communication
    def _global(self, r: int) -> int:
        return r if self.group is None else dist.get_global_rank(self.group, r)

    def _exchange(self, send: Sequence[torch.Tensor], send_to: Optional[int],
                  recv: Sequence[torch.Tensor], recv_from: Optional[int]) -> None:
        """Posts every send / receive slab as one batch and waits; a peer that never joins makes the wait
        fail after the process group's timeout, reported as PeerExchangeError."""
        check_peers(self.store)
        ops = []
        if send_to is not None:
            ops += [dist.P2POp(dist.isend, t, self._global(send_to), self.group) for t in send]
        if recv_from is not None:
            ops += [dist.P2POp(dist.irecv, t, self._global(recv_from), self.group) for t in recv]
        if not ops:
            return
        try:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        except PeerExchangeError:
            raise
        except Exception as e:       # noqa: BLE001 -- backend-specific error types (timeouts, closed connections)
            raise PeerExchangeError(f"rank {self.rank}: exchange with ranks {send_to}/{recv_from} failed: {e}") from e

    def _halo_rows_for_right(self) -> int:
        """Rows this rank sends to its right neighbour (that neighbour's halo length)."""
        if self.plan.right is None:
            return 0
        return min(RING, self.shards[self.plan.right][0])

    @staticmethod
    def _slabs(t: torch.Tensor, rows: slice) -> list[torch.Tensor]:
        """Contiguous [rows, D] pieces of t[..., rows, :] (t is [..., N, D] contiguous): one per leading index."""
        flat = t.reshape(-1, t.shape[-2], t.shape[-1])
        return [flat[i, rows] for i in range(flat.shape[0])]

    # ------------------------------------------------------------------ local buffers
    def local_buffers(self, B: int, Hq: int, Hkv: int, D: int, dtype, device):
        """Allocates (once) and returns views (Q, R, S, Vr, Vs, dY) of this rank's own rows inside the local
        buffers.  A caller that writes its shards there and passes these views to forward/backward saves the
        copies into the buffers."""
        p = self.plan
        n_loc = p.halo + (p.hi - p.lo) + p.pad
        if self._kv is None or self._kv.shape != (4, B, Hkv, n_loc, D) or self._kv.dtype != dtype:
            self._kv = torch.zeros(4, B, Hkv, n_loc, D, dtype=dtype, device=device)
            self._q = torch.zeros(B, Hq, n_loc, D, dtype=dtype, device=device)
            self._dy = torch.zeros(B, Hq, n_loc, D, dtype=dtype, device=device)
        own = slice(p.halo, p.halo + (p.hi - p.lo))
        return (self._q[:, :, own], self._kv[0][:, :, own], self._kv[1][:, :, own], self._kv[2][:, :, own],
                self._kv[3][:, :, own], self._dy[:, :, own])

    @staticmethod
    def _same(view: torch.Tensor, t: torch.Tensor) -> bool:
        return t.data_ptr() == view.data_ptr() and t.shape == view.shape and t.stride() == view.stride()

    # ------------------------------------------------------------------ forward
    def forward(self, Q, R, S, Vr, Vs):
        """Local shards [B,H*,hi-lo,D] -> local Y [B,Hq,hi-lo,D] (and statistics kept for backward)."""
        p = self.plan
        if p.hi <= p.lo:
            self._saved = None
            self._exchange([], None, [], None)
            return Q.new_zeros(Q.shape)
        n_own = p.hi - p.lo
        views = self.local_buffers(Q.shape[0], Q.shape[1], R.shape[1], Q.shape[3], Q.dtype, Q.device)
        for view, t in zip(views[:5], (Q, R, S, Vr, Vs)):
            if not self._same(view, t):
                view.copy_(t)
        kv = self._kv
        n_send = self._halo_rows_for_right()
        send = self._slabs(kv, slice(p.halo + n_own - n_send, p.halo + n_own)) if n_send else []
        recv = self._slabs(kv, slice(0, p.halo)) if p.halo else []
        self._exchange(send, p.right, recv, p.left)
        Y, m, l = self._fwd(self._q, kv[0], kv[1], kv[2], kv[3], self.window, p.halo)
        self._saved = (Y, m, l)
        return Y[:, :, p.halo:p.halo + n_own]

    # ------------------------------------------------------------------ backward
    def backward(self, dY):
        """Local cotangent [B,Hq,hi-lo,D] -> (dQ, dR, dS, dVr, dVs) for the local rows, with the
        contributions of the right neighbour's queries to this rank's last rows added in (in FP32,
        before the one rounding to the input dtype)."""
        p = self.plan
        n_own = p.hi - p.lo
        if n_own <= 0 or self._saved is None:
            z = dY.new_zeros(dY.shape)
            return z, None, None, None, None
        Y, m, l = self._saved
        dy_view = self.local_buffers(dY.shape[0], dY.shape[1], self._kv.shape[2], dY.shape[3], dY.dtype, dY.device)[5]
        if not self._same(dy_view, dY):
            dy_view.copy_(dY)
        kv = self._kv
        dQ, dR, dS, dVr, dVs = self._bwd(self._dy, self._q, kv[0], kv[1], kv[2], kv[3], Y, m, l, self.window, p.halo)
        grads = [dR, dS, dVr, dVs]
        acc = torch.promote_types(dR.dtype, torch.float32)
        if any(g.dtype != acc for g in grads):                   # a compute step that rounded already: widen
            grads = [g.to(acc) for g in grads]
        send = [s for g in grads for s in self._slabs(g, slice(0, p.halo))] if p.halo else []
        n_recv = self._halo_rows_for_right()
        recv_buf = grads[0].new_empty(4, *dR.shape[:2], n_recv, dR.shape[3]) if n_recv else None
        recv = self._slabs(recv_buf, slice(0, n_recv)) if n_recv else []
        self._exchange(send, p.left, recv, p.right)
        out = []
        for k, g in enumerate(grads):
            own = g[:, :, p.halo:p.halo + n_own]
            if n_recv:
                own = own.clone()
                own[:, :, n_own - n_recv:] += recv_buf[k]
            out.append(own.to(kv.dtype))
        return (dQ[:, :, p.halo:p.halo + n_own], *out)


class HeadShardedGather:
    """Shared-KV single gather with the query heads of each KV head split over the ranks of `group`
    (the second axis of the (batch, head) partition: batches go to different groups, the heads of one
    batch to the ranks of one group).  Rank r holds Q[:, heads_r] and dY[:, heads_r] and the whole key
    side R, S, Vr, Vs ([B,Hkv,N,D], the same on every rank of the group).

    The forward is local.  In the backward dQ is local, while every rank's key-side gradients are sums
    over its own heads only: the FP32 partials are summed over the group with one all-reduce per key
    side (2 x [B,Hkv,N,D] floats each) and rounded once afterwards -- the reduction the reference
    performs over its per-head partial buffers inside one GPU (cuda/backward.cu:2548-2575), done across
    GPUs.  The first side's all-reduce is issued as soon as that side is complete and runs on the
    communicator's stream while the second side is computed.

    ``compute_fwd(Q,R,S,Vr,Vs,window) -> (Y,m,l)``; ``compute_bwd(dY,Q,R,S,Vr,Vs,Y,m,l,window,between)
    -> (dQ, kv32)`` with kv32 = FP32 [4,B,Hkv,N,D] holding dS, dVs, dR, dVr and ``between(kv32[:2])``
    called once the first two are complete.  Both default to the CUDA kernels."""

    def __init__(self, window: int, group=None, compute_fwd: Optional[Callable] = None,
                 compute_bwd: Optional[Callable] = None, store=None):
        if not 1 <= window <= RING:
            raise ValueError(f"window must be in [1,{RING}], got {window}")
        self.group, self.window, self.store = group, window, store
        if compute_fwd is None or compute_bwd is None:
            from . import _cuda_kernels as ck
            compute_fwd = compute_fwd or (lambda Q, R, S, Vr, Vs, w: ck.sg_forward_raw(Q, R, S, Vr, Vs, None, w))
            compute_bwd = compute_bwd or (lambda dY, Q, R, S, Vr, Vs, Y, m, l, w, between:
                                          ck.sg_backward_sides_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w,
                                                                   between=between))
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
        check_peers(self.store)
        pending = []

        alone = dist.get_world_size(self.group) == 1          # all heads here: nothing to sum

        def start_reduce(part):
            if not alone:
                pending.append(dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group, async_op=True))

        try:
            dQ, kv32 = self._bwd(dY, Q, R, S, Vr, Vs, Y, m, l, self.window, start_reduce)
            start_reduce(kv32[2:])
            for work in pending:
                work.wait()
        except PeerExchangeError:
            raise
        except Exception as e:       # noqa: BLE001 -- backend-specific error types
            raise PeerExchangeError(f"key-gradient all-reduce failed: {e}") from e
        kv = kv32.to(out_dtype or R.dtype)
        return dQ, kv[2], kv[0], kv[3], kv[1]


def gather_rows(local: torch.Tensor, shards: Sequence[tuple[int, int]], group=None) -> torch.Tensor:
    """All-gathers row shards (dim 2) into the full tensor on every rank; for tests and checks."""
    world = dist.get_world_size(group)
    longest = max(hi - lo for lo, hi in shards)
    buf = torch.nn.functional.pad(local, (0, 0, 0, longest - local.size(2))).contiguous()
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf, group=group)
    return torch.cat([parts[r][:, :, :hi - lo] for r, (lo, hi) in enumerate(shards)], dim=2)
