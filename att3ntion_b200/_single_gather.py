"""Autograd bridge of the Q-anchored single gather,

    Y[i] = sum_{j,k} softmax_{(j,k)}(Q_i . R_j . S_k / sqrt(D)) Vr[j] o Vs[k]

with the call signature and padding rules of the reference bridge
(att3ntion/_single_gather.py:28-70): inputs are cast to BF16, N is padded to a
multiple of 16 with padded positions invisible as queries and as keys, the
result is cropped and cast back.  Differences, both invisible to callers:
an equal causal window (``window`` in 1..128, no extra mask) is generated from
indices inside the kernel instead of being materialised as a [B,N,N] tensor,
and the padding rows of such a call need no mask either, because a causal
window never lets a real query see a later (padded) key.  A mask that comes with
such a window is packed into words once per forward (1/32 of the bytes) and the
words serve the forward and the backward.  Beyond the reference: ``window`` may be
a pair (w_r, w_s), one causal window per key axis (the reference lists independent
windows as an open item, docs/KERNEL_HISTORY.md:180).
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


def _window_pair(window, n: int):
    """(w_r, w_s) from an int or a pair, each clipped to the sequence length (>= N: causal); 0 = no window."""
    if isinstance(window, (tuple, list)):
        if len(window) != 2:
            raise ValueError("single_gather_attention: window is an int or a pair (w_r, w_s)")
        wr, ws = int(window[0]), int(window[1])
        if (wr > 0) != (ws > 0):
            raise ValueError("single_gather_attention: a pair of windows needs both positive")
    else:
        wr = ws = int(window) if window else 0
    return (min(wr, n) if wr else 0), (min(ws, n) if ws else 0)


class _SingleGatherFn(Function):
    @staticmethod
    def forward(ctx, Q, R, S, Vr, Vs, mask, window, precise=False):
        n = Q.size(2)
        n_pad = (-n) % TILE
        xs = [_pad_rows(x.contiguous().to(torch.bfloat16), n_pad) for x in (Q, R, S, Vr, Vs)]
        window, window_s = _window_pair(window, n)
        ring = 0 < window <= 128 and 0 < window_s <= 128
        if (window or window_s) and not ring:
            if window != window_s:
                raise ValueError("single_gather_attention: a pair of windows needs both in 1..128")
            if mask is None:
                mask = window_mask(n, window, Q.device)      # wider than the resident ring: dense schedule
        if mask is None and n_pad and not ring:
            mask = torch.ones(Q.size(0), n, n, dtype=torch.bool, device=Q.device)
        mask = _prepare_mask(mask, Q.size(0), n, n_pad, Q.device)
        win = window if ring else 0
        win_s = window_s if (ring and window_s != window) else 0
        if precise and not ring:
            raise ValueError("single_gather_attention: precise=True needs a causal window in 1..128")
        words = None
        if ring and mask is not None:
            words, mask = _ck.pack_mask(mask), None          # the window itself comes from indices inside the kernels
        Y, m, l = _ck.sg_forward_raw(*xs, mask, win, 0, win_s, words, precise=bool(precise))
        keep = words if words is not None else (mask if mask is not None else torch.empty(0))
        ctx.save_for_backward(*xs, Y, m, l, keep)
        ctx.n, ctx.dtype, ctx.win, ctx.win_s, ctx.packed = n, Q.dtype, win, win_s, words is not None
        ctx.precise = bool(precise)
        return Y[:, :, :n].to(Q.dtype)

    @staticmethod
    def backward(ctx, dY):
        Q, R, S, Vr, Vs, Y, m, l, keep = ctx.saved_tensors
        mask = keep if (keep.numel() and not ctx.packed) else None
        words = keep if ctx.packed else None
        dY = _pad_rows(dY.contiguous().to(torch.bfloat16), Q.size(2) - ctx.n)
        grads = _ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, mask, ctx.win, 0, False, ctx.win_s, words,
                                    precise=ctx.precise)
        return tuple(g[:, :, :ctx.n].to(ctx.dtype) for g in grads) + (None, None, None)


def single_gather_attention(Q, R, S, Vr, Vs, mask=None, window=0, *, precise=False):
    """Q, R, S, Vr, Vs: [B,H,N,D] with D in {64,128}.  mask: [B,N,N] or [N,N] bool,
    True = visible; query i attends the pairs (j,k) whose members are both visible
    to it, and a fully masked query returns zeros.  window > 0 declares an equal
    causal window of that width on both key axes (>= N: causal); with no mask the
    window is the visibility, with a mask the two are intersected.  window = (w_r, w_s)
    gives the R / Vr axis and the S / Vs axis a causal window each (both in 1..128).
    precise=True (windows in 1..128 only) runs the score products on the exact split of
    Q o R into its BF16 value and residual: scores of large magnitude, whose BF16 rounding
    the softmax would amplify, keep FP32 accuracy at 1.8x the time (the
    reference's unshipped "compensated" path, docs/KERNEL_HISTORY.md:22)."""
    return _SingleGatherFn.apply(Q, R, S, Vr, Vs, mask, window, precise)


class _SingleGatherHeadsLastFn(Function):
    """The windowed gather on operands laid out [B,N,H,D] -- the projections' own output viewed as heads -- with
    the module's activation optionally taken from the forward's epilogue.  The reference's module permutes every
    operand to [B,H,N,D] and copies it before the op, and runs QuickGELU as a separate pass afterwards
    (att3ntion/_autograd.py:349-363, 395-403); none of that happens here."""

    @staticmethod
    def forward(ctx, Q, R, S, Vr, Vs, window, act):
        xs = [x.contiguous().to(torch.bfloat16) for x in (Q, R, S, Vr, Vs)]
        out = _ck.sg_forward_raw(*xs, None, int(window), bnhd=True, act=bool(act))
        Y, m, l = out[:3]
        ctx.save_for_backward(*xs, Y, m, l)
        ctx.window, ctx.act, ctx.dtype = int(window), bool(act), Q.dtype
        return (out[3] if act else Y).to(Q.dtype)

    @staticmethod
    def backward(ctx, dOut):
        Q, R, S, Vr, Vs, Y, m, l = ctx.saved_tensors
        dOut = dOut.contiguous()
        if ctx.act:
            # d/dy [y sigmoid(a y)] = s (1 + a y (1 - s)), s = sigmoid(a y), a = 1.702
            y = Y.float()
            sg = torch.sigmoid(1.702 * y)
            dY = (dOut.float() * sg * (1.0 + 1.702 * y * (1.0 - sg))).to(torch.bfloat16)
        else:
            dY = dOut.to(torch.bfloat16)
        grads = _ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, ctx.window, bnhd=True)
        return tuple(g.to(ctx.dtype) for g in grads) + (None, None)


def single_gather_heads_last(Q, R, S, Vr, Vs, window, act=False):
    """Q [B,N,Hq,D], R, S, Vr, Vs [B,N,Hkv,D] (Hq a multiple of Hkv), D in {64,128}, N a multiple of 16, causal
    window in 1..128 on both key axes and no extra mask.  Returns Y, or QuickGELU(Y) with act=True, as [B,N,Hq,D]."""
    n = Q.size(1)
    if n % TILE or not 0 < int(window) <= 128:
        raise ValueError("single_gather_heads_last: needs N % 16 == 0 and a window in 1..128")
    return _SingleGatherHeadsLastFn.apply(Q, R, S, Vr, Vs, min(int(window), n), act)
