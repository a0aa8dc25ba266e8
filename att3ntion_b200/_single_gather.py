"""Autograd bridge of the Q-anchored single gather,

    Y[i] = sum_{j,k} softmax_{(j,k)}(Q_i . R_j . S_k / sqrt(D)) Vr[j] o Vs[k]

with the call signature and padding rules of the reference bridge
(att3ntion/_single_gather.py:28-70): inputs are cast to BF16, N is padded to a
multiple of 16 with padded positions invisible as queries and as keys, the
result is cropped and cast back.  Differences, both invisible to callers:
an equal causal window (``window`` in 1..128, no extra mask) is generated from
indices inside the kernel instead of being materialised as a [B,N,N] tensor,
and the padding rows of such a call need no mask either, because a causal
window never lets a real query see a later (padded) key.
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import _cuda_kernels as _ck

TILE = 16


def _pad_rows(t: torch.Tensor, n_pad: int) -> torch.Tensor:
    return torch.nn.functional.pad(t, (0, 0, 0, n_pad)) if n_pad else t


def window_mask(n: int, window: int, device) -> torch.Tensor:
    """[n,n] bool: query i sees key j iff i - window < j <= i (window >= n: causal)."""
    i = torch.arange(n, device=device)
    return (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - window)


def _prepare_mask(mask, batch: int, n: int, n_pad: int, device):
    """Bool [B, n+n_pad, n+n_pad] with the padding invisible, or None."""
    if mask is None:
        return None
    mask = mask.to(device=device, dtype=torch.bool)
    if mask.dim() == 2:
        mask = mask.unsqueeze(0)
    if mask.size(0) == 1 and batch > 1:
        mask = mask.expand(batch, -1, -1)
    return torch.nn.functional.pad(mask, (0, n_pad, 0, n_pad), value=False).contiguous()


class _SingleGatherFn(Function):
    @staticmethod
    def forward(ctx, Q, R, S, Vr, Vs, mask, window):
        n = Q.size(2)
        n_pad = (-n) % TILE
        xs = [_pad_rows(x.contiguous().to(torch.bfloat16), n_pad) for x in (Q, R, S, Vr, Vs)]
        window = min(int(window), n) if window else 0
        ring = 0 < window <= 128
        if window and not ring and mask is None:
            mask = window_mask(n, window, Q.device)          # wider than the resident ring: dense schedule
        if mask is None and n_pad and not ring:
            mask = torch.ones(Q.size(0), n, n, dtype=torch.bool, device=Q.device)
        mask = _prepare_mask(mask, Q.size(0), n, n_pad, Q.device)
        win = window if ring else 0
        Y, m, l = _ck.sg_forward_raw(*xs, mask, win)
        ctx.save_for_backward(*xs, Y, m, l, mask if mask is not None else torch.empty(0))
        ctx.n, ctx.dtype, ctx.win = n, Q.dtype, win
        return Y[:, :, :n].to(Q.dtype)

    @staticmethod
    def backward(ctx, dY):
        Q, R, S, Vr, Vs, Y, m, l, mask = ctx.saved_tensors
        mask = mask if mask.numel() else None
        dY = _pad_rows(dY.contiguous().to(torch.bfloat16), Q.size(2) - ctx.n)
        grads = _ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, mask, ctx.win)
        return tuple(g[:, :, :ctx.n].to(ctx.dtype) for g in grads) + (None, None)


def single_gather_attention(Q, R, S, Vr, Vs, mask=None, window=0):
    """Q, R, S, Vr, Vs: [B,H,N,D] with D in {64,128}.  mask: [B,N,N] or [N,N] bool,
    True = visible; query i attends the pairs (j,k) whose members are both visible
    to it, and a fully masked query returns zeros.  window > 0 declares an equal
    causal window of that width on both key axes (>= N: causal); with no mask the
    window is the visibility, with a mask the two are intersected."""
    return _SingleGatherFn.apply(Q, R, S, Vr, Vs, mask, window)
