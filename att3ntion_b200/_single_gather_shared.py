"""Autograd bridge of the shared-KV single gather: the operator of
``single_gather_attention`` with R, S, Vr, Vs shared by every query head
([B,1,N,128]) and read in place.  Signature and contract follow the reference
bridge (att3ntion/_single_gather_shared.py:19-60): D = 128, one KV head, an
equal causal window of 16, 32, 64 or 128, an optional mask that may only remove
pairs inside that window, N padded to a multiple of 16, KV gradients returned
as [B,1,N,128] (summed over query heads).

The reference materialises the window as a dense [B,N,N] bool tensor on every
call; here the kernels derive it from indices, and only a caller-supplied extra
mask is passed on, packed into one bit per key (the form of the reference's mask
metadata, cuda/shared_kv/shared_mask_metadata.cuh:8-31).
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import _cuda_kernels as _ck
from ._single_gather import TILE, _pad_rows, _prepare_mask

WINDOW = 128


class _SharedFn(Function):
    @staticmethod
    def forward(ctx, Q, R, S, Vr, Vs, mask, fwd_group, rs_group, window, precise=False):
        n = Q.size(2)
        n_pad = (-n) % TILE
        xs = [_pad_rows(x.contiguous().to(torch.bfloat16), n_pad) for x in (Q, R, S, Vr, Vs)]
        _ck._check_shared(xs[0], xs[1:], None, window, 1 if fwd_group == 0 else fwd_group, need_mask=False)
        _ck._check_shared(xs[0], xs[1:], None, window, 1 if rs_group == 0 else rs_group, need_mask=False)
        mask = _prepare_mask(mask, Q.size(0), n, n_pad, Q.device)
        # an extra mask is packed into words once (1/32 of the bytes) and serves the forward and the backward
        words = _ck.pack_mask(mask) if mask is not None else None
        Y, m, l = _ck.sg_forward_raw(*xs, None, window, 0, 0, words, precise=bool(precise))
        ctx.save_for_backward(*xs, Y, m, l, words if words is not None else torch.empty(0))
        ctx.n, ctx.dtype, ctx.window, ctx.precise = n, Q.dtype, window, bool(precise)
        return Y[:, :, :n].to(Q.dtype)

    @staticmethod
    def backward(ctx, dY):
        Q, R, S, Vr, Vs, Y, m, l, words = ctx.saved_tensors
        words = words if words.numel() else None
        dY = _pad_rows(dY.contiguous().to(torch.bfloat16), Q.size(2) - ctx.n)
        grads = _ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, ctx.window, 0, False, 0, words,
                                    precise=ctx.precise)
        return tuple(g[:, :, :ctx.n].to(ctx.dtype) for g in grads) + (None, None, None, None, None)


def single_gather_shared_attention(Q, R, S, Vr, Vs, mask=None, fwd_group=0, rs_group=0, window=WINDOW, *, precise=False):
    """Q: [B,Hq,N,128]; R, S, Vr, Vs: [B,1,N,128].  Causal `window` (16, 32, 64 or
    128) on both key axes, optionally narrowed by `mask` ([B,N,N] or [N,N] bool).

    fwd_group / rs_group exist for call compatibility (0, 1, 2 or 4; Hq must be
    divisible by a non-zero group): the sm_100a kernels always let one CTA walk
    all query heads of a KV head, so every value runs the same schedule and gives
    bit-identical results.  A query with a single visible key gets exactly zero
    score gradients.  Inputs and dY are cast to BF16; accumulation is FP32.  precise=True: score
    products on the exact value + residual split of Q o R (see single_gather_attention)."""
    return _SharedFn.apply(Q, R, S, Vr, Vs, mask, fwd_group, rs_group, window, precise)
