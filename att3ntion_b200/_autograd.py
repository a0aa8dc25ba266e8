"""``HypergraphAttention`` and its autograd bridge, API-compatible with the reference
module (att3ntion/_autograd.py:12-405): same constructor arguments, parameter names
and shapes (so state dicts load either way), same forward semantics

    y = Wo( gelu(Y_q) + gelu(Y_r) + gelu(Y_s) [+ the three scatter terms] )

with QuickGELU, heads split from ``d_model``, inputs cast to BF16 at the kernel
boundary and the sequence padded to a multiple of 16 with the padding invisible.
``gather_mode=1`` keeps only the Q-anchored gather and, for head sizes 64 and 128,
routes to ``single_gather_attention`` (optionally windowed).
"""
from __future__ import annotations

import os

import torch
import torch.nn as nn
from torch.autograd import Function

from . import _custom_op  # noqa: F401  (registers torch.ops.att3ntion.hypergraph_{forward,backward})
from ._single_gather import single_gather_attention, single_gather_heads_last, window_mask

TILE = 16
_CHECK_GRADS = os.getenv("ATT3NTION_CHECK_GRADS", "0").lower() in {"1", "true", "yes", "on"}


def _pad_to_multiple(t: torch.Tensor, multiple: int, dim: int = 2):
    """Right-pads `dim` of `t` with zeros to a multiple of `multiple`; returns (tensor, pad)."""
    extra = (-t.size(dim)) % multiple
    if extra == 0:
        return t, 0
    pad = [0, 0] * t.ndim
    pad[2 * (t.ndim - 1 - dim) + 1] = extra          # F.pad lists dims from the last one backwards
    return torch.nn.functional.pad(t, pad), extra


def _normalize_self_attn_mask(mask, batch: int, n: int, device):
    """None, or a contiguous bool [batch, n, n] on `device` from a [n,n] / [1,n,n] / [batch,n,n] mask."""
    if mask is None:
        return None
    if mask.ndim == 2:
        if tuple(mask.shape) != (n, n):
            raise ValueError(f"2D mask must have shape {(n, n)}, got {tuple(mask.shape)}")
        mask = mask.unsqueeze(0)
    elif mask.ndim != 3:
        raise ValueError(f"mask must have ndim 2 or 3, got ndim={mask.ndim}")
    if tuple(mask.shape[-2:]) != (n, n):
        raise ValueError(f"mask must have trailing shape {(n, n)}, got {tuple(mask.shape)}")
    if mask.shape[0] not in (1, batch):
        raise ValueError(f"mask batch dim must be 1 or {batch}, got {mask.shape[0]}")
    if mask.shape[0] == 1 and batch > 1:
        mask = mask.expand(batch, -1, -1)
    return mask.to(device=device, dtype=torch.bool).contiguous()


class _HypergraphAttentionAutograd(Function):
    """Casts and pads at the kernel boundary, calls the registered ops, crops and casts back."""

    @staticmethod
    def forward(ctx, Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2, mask, dropout_rate=0.0, scatter=False,
                gather_mode=0):
        n = Q.size(2)
        if mask is not None and (R.size(2) != n or S.size(2) != n):
            raise ValueError("masked CUDA hypergraph attention requires equal sequence lengths")
        mask = _normalize_self_attn_mask(mask, Q.size(0), n, Q.device)
        xs = [_pad_to_multiple(t.contiguous().to(torch.bfloat16), TILE)[0]
              for t in (Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2)]
        n_pad = xs[0].size(2) - n
        if mask is None:
            mask_t = torch.empty(0, device=Q.device, dtype=torch.bool)
        else:
            mask_t = torch.nn.functional.pad(mask, (0, n_pad, 0, n_pad), value=False).contiguous() if n_pad else mask
        out = torch.ops.att3ntion.hypergraph_forward(*xs, mask_t, float(dropout_rate), n, n, n, int(gather_mode))
        Ys, stats = out[:6], out[6:]
        ctx.save_for_backward(*xs, *stats, mask_t, *Ys[:3])
        ctx.n, ctx.dtype = n, Q.dtype
        return tuple(y[:, :, :n].to(Q.dtype) for y in Ys)

    @staticmethod
    def backward(ctx, *cot):
        saved = ctx.saved_tensors
        xs, stats, mask_t, Y3 = saved[:9], saved[9:15], saved[15], saved[16:19]
        n_full = xs[0].size(2)
        gs = []
        for g, y in zip(cot, (*Y3, *Y3)):
            if g is None:
                gs.append(torch.zeros_like(y))
            else:
                gs.append(_pad_to_multiple(g.contiguous().to(torch.bfloat16), TILE)[0])
        grads = torch.ops.att3ntion.hypergraph_backward(*gs, *xs, *stats, mask_t, *Y3)
        grads = [g[:, :, :ctx.n].to(ctx.dtype) if n_full != ctx.n else g.to(ctx.dtype) for g in grads]
        if _CHECK_GRADS:
            for name, g in zip(("Q", "R", "S", "Vq_1", "Vq_2", "Vr_1", "Vr_2", "Vs_1", "Vs_2"), grads):
                if not torch.isfinite(g).all():
                    raise RuntimeError(f"grad_{name} contains non-finite values")
        return (*grads, None, None, None, None)


class QuickGELU(nn.Module):
    def forward(self, x: torch.Tensor):
        return x * torch.sigmoid(1.702 * x)


class HypergraphAttention(nn.Module):
    """Three-way hypergraph attention layer on the sm_100a kernels."""

    def __init__(self, d_model, n_heads, dropout_rate=0, scatter=False, gather_mode=0, window=0):
        super().__init__()
        if d_model % n_heads != 0:
            raise ValueError(f"d_model ({d_model}) must be divisible by n_heads ({n_heads})")
        if gather_mode not in (0, 1):
            raise ValueError(f"gather_mode must be 0 (Q, R and S anchored) or 1 (Q anchored only), got {gather_mode}")
        if scatter and gather_mode != 0:
            raise ValueError("scatter requires all three gathers (gather_mode=0)")
        if window and gather_mode != 1:
            raise ValueError("window requires the Q-anchored gather only (gather_mode=1)")
        self.d_model, self.n_heads, self.head_dim = d_model, n_heads, d_model // n_heads
        self.scatter, self.gather_mode, self.window = scatter, gather_mode, window
        inner = n_heads * self.head_dim
        self.Wq = nn.Linear(d_model, inner, bias=False)
        self.Wr = nn.Linear(d_model, inner, bias=False)
        self.Ws = nn.Linear(d_model, inner, bias=False)
        vmul = 2 if scatter else 1
        # the Q-anchored gather never reads Vq, so the one-gather variant has no Wv_q
        self.Wv_q = None if gather_mode == 1 else nn.Linear(d_model, inner * vmul, bias=True)
        self.Wv_r = nn.Linear(d_model, inner * vmul, bias=True)
        self.Wv_s = nn.Linear(d_model, inner * vmul, bias=True)
        self.Wo = nn.Linear(inner, d_model, bias=True)
        self.dropout = nn.Dropout(dropout_rate)
        self.gelu = QuickGELU()

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        # value projections saved with / without the scatter half load into either configuration
        for name in ("Wv_q", "Wv_r", "Wv_s"):
            module = getattr(self, name)
            if module is None:
                continue
            for suffix, target in (("weight", module.weight), ("bias", module.bias)):
                key = f"{prefix}{name}.{suffix}"
                loaded = state_dict.get(key)
                if loaded is None or loaded.shape == target.shape or loaded.ndim != target.ndim:
                    continue
                if loaded.shape[0] == 2 * target.shape[0] and loaded.shape[1:] == target.shape[1:]:
                    state_dict[key] = loaded[: target.shape[0]].contiguous()
                elif 2 * loaded.shape[0] == target.shape[0] and loaded.shape[1:] == target.shape[1:]:
                    grown = torch.zeros_like(target)
                    grown[: loaded.shape[0]] = loaded
                    state_dict[key] = grown
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)

    def _heads(self, t, width=None):
        b, n, _ = t.shape
        return t.reshape(b, n, self.n_heads, width or self.head_dim).permute(0, 2, 1, 3)

    def forward(self, x, rotary_emb=None, mask=None):
        if rotary_emb is not None:
            raise ValueError("CUDA HypergraphAttention does not support rotary embeddings")
        b, n, _ = x.shape
        Q, R, S = self.Wq(x), self.Wr(x), self.Ws(x)
        window_only = bool(self.window) and mask is None      # then the kernels derive the window from indices
        if self.window:
            win = window_mask(n, self.window, x.device)
            mask = win if mask is None else mask.to(device=x.device, dtype=torch.bool) & win

        if self.gather_mode == 1 and self.head_dim in (64, 128) and window_only and self.window <= 128 and n % TILE == 0:
            # window-only calls read the projections where they lie ([B,N,H,D] views, no permute-and-copy) and take
            # the activation from the kernel's epilogue
            split = lambda t: t.view(b, n, self.n_heads, self.head_dim)
            y = single_gather_heads_last(split(Q), split(R), split(S), split(self.Wv_r(x)), split(self.Wv_s(x)),
                                         min(self.window, n), act=True)
            return self.Wo(y.reshape(b, n, self.n_heads * self.head_dim))

        if self.gather_mode == 1 and self.head_dim in (64, 128):
            y = single_gather_attention(self._heads(Q), self._heads(R), self._heads(S), self._heads(self.Wv_r(x)),
                                        self._heads(self.Wv_s(x)), None if window_only else mask,
                                        min(self.window, n))
            y = self.gelu(y).permute(0, 2, 1, 3).contiguous().view(b, n, self.n_heads * self.head_dim)
            return self.Wo(y)

        if self.scatter:
            Vq_1, Vq_2 = self._heads(self.Wv_q(x), 2 * self.head_dim).split(self.head_dim, dim=-1)
            Vr_1, Vr_2 = self._heads(self.Wv_r(x), 2 * self.head_dim).split(self.head_dim, dim=-1)
            Vs_1, Vs_2 = self._heads(self.Wv_s(x), 2 * self.head_dim).split(self.head_dim, dim=-1)
        else:
            Vr_1, Vs_1 = self._heads(self.Wv_r(x)), self._heads(self.Wv_s(x))
            Vq_1 = torch.zeros_like(Vr_1) if self.Wv_q is None else self._heads(self.Wv_q(x))
            Vq_2, Vr_2, Vs_2 = torch.zeros_like(Vq_1), torch.zeros_like(Vr_1), torch.zeros_like(Vs_1)

        Y_q, Y_r, Y_s, Y_q_, Y_r_, Y_s_ = _HypergraphAttentionAutograd.apply(
            self._heads(Q), self._heads(R), self._heads(S), Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2, mask,
            self.dropout.p, self.scatter, self.gather_mode)
        y = self.gelu(Y_q)
        if self.gather_mode == 0:
            y = y + self.gelu(Y_r) + self.gelu(Y_s)
        if self.scatter:
            y = y + self.gelu(Y_q_) + self.gelu(Y_r_) + self.gelu(Y_s_)
        y = y.permute(0, 2, 1, 3).contiguous().view(b, n, self.n_heads * self.head_dim)
        return self.Wo(y)
