"""torch.library registration of the three-gather operator, with the schema of the
reference (att3ntion/_custom_op.py:23-154): ``att3ntion::hypergraph_forward`` returns
six outputs and six statistics, ``att3ntion::hypergraph_backward`` nine gradients;
both have fake (meta) kernels so ``torch.compile`` can trace through them, and the
forward op has an autograd formula that calls the backward op.  "No mask" is an
empty bool tensor at this level (att3ntion/_autograd.py:106-107).
"""
from __future__ import annotations

import torch
from torch.library import custom_op

from . import _cuda_kernels as _ck

T = torch.Tensor


@custom_op("att3ntion::hypergraph_forward", mutates_args=())
def hypergraph_forward(Q: T, R: T, S: T, Vq_1: T, Vq_2: T, Vr_1: T, Vr_2: T, Vs_1: T, Vs_2: T, mask: T,
                       dropout_rate: float, I_valid: int = -1, J_valid: int = -1, K_valid: int = -1,
                       gather_mode: int = 0) -> tuple[T, T, T, T, T, T, T, T, T, T, T, T]:
    return _ck.forward(Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2, dropout_rate, I_valid, J_valid, K_valid,
                       mask if mask.numel() else None, gather_mode)


@hypergraph_forward.register_fake
def _forward_fake(Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2, mask, dropout_rate, I_valid=-1, J_valid=-1,
                  K_valid=-1, gather_mode=0):
    B, H, _, D = Q.shape
    outs = [torch.empty((B, H, t.shape[2], D), dtype=Q.dtype, device=Q.device) for t in (Q, R, S, Q, R, S)]
    stats = [torch.empty((B, H, t.shape[2]), dtype=torch.float32, device=Q.device) for t in (Q, Q, R, R, S, S)]
    return (*outs, *stats)


@custom_op("att3ntion::hypergraph_backward", mutates_args=())
def hypergraph_backward(grad_Y_q: T, grad_Y_r: T, grad_Y_s: T, grad_Y_q_: T, grad_Y_r_: T, grad_Y_s_: T,
                        Q: T, R: T, S: T, Vq_1: T, Vq_2: T, Vr_1: T, Vr_2: T, Vs_1: T, Vs_2: T,
                        m_i: T, l_i: T, m_j: T, l_j: T, m_k: T, l_k: T, mask: T,
                        Y_q: T, Y_r: T, Y_s: T) -> tuple[T, T, T, T, T, T, T, T, T]:
    return _ck.backward(grad_Y_q, grad_Y_r, grad_Y_s, grad_Y_q_, grad_Y_r_, grad_Y_s_, Q, R, S,
                        Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2, m_i, l_i, m_j, l_j, m_k, l_k, 0.0,
                        mask if mask.numel() else None, Y_q, Y_r, Y_s)


@hypergraph_backward.register_fake
def _backward_fake(grad_Y_q, grad_Y_r, grad_Y_s, grad_Y_q_, grad_Y_r_, grad_Y_s_, Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2,
                   Vs_1, Vs_2, m_i, l_i, m_j, l_j, m_k, l_k, mask, Y_q, Y_r, Y_s):
    return tuple(torch.empty_like(t) for t in (Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2))


def _setup_context(ctx, inputs, output):
    Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2, mask = inputs[:10]
    Y_q, Y_r, Y_s, _, _, _, m_i, l_i, m_j, l_j, m_k, l_k = output
    ctx.save_for_backward(Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2, m_i, l_i, m_j, l_j, m_k, l_k, mask,
                          Y_q, Y_r, Y_s)


def _backward(ctx, gq, gr, gs, gq_, gr_, gs_, *_stats):
    (Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2, m_i, l_i, m_j, l_j, m_k, l_k, mask, Y_q, Y_r, Y_s) = ctx.saved_tensors
    cot = [torch.zeros_like(y) if g is None else g.contiguous().to(torch.bfloat16)
           for g, y in zip((gq, gr, gs, gq_, gr_, gs_), (Y_q, Y_r, Y_s, Y_q, Y_r, Y_s))]
    grads = torch.ops.att3ntion.hypergraph_backward(*cot, Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2,
                                                    m_i, l_i, m_j, l_j, m_k, l_k, mask, Y_q, Y_r, Y_s)
    return (*grads, None, None, None, None, None, None)


hypergraph_forward.register_autograd(_backward, setup_context=_setup_context)
