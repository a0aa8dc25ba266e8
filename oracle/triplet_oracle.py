"""CPU oracle for the triplet (hypergraph) attention hot path.  TEST INFRASTRUCTURE.

This module restates, in plain FP64 torch on the CPU, the arithmetic that the
CUDA kernels of this repository must reproduce.  It is the checker: only the
test-suite, the smoke check and the CPU-baseline leg of the benchmark may import
it.  No product code path routes through it.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference's
own oracles (tests/test_single_gather.py:52-66 ``reference``; the masked
three-gather rule of tests/test_tc_paths.py:218-238; cpp/torch_reference.cpp:24-57
through att3ntion/_naive.py) in a container that has the reference mounted, runs
them on seeded inputs and commits the outputs under ``tests/golden``;
``tests/test_oracle_golden.py`` checks every function here against those files.

What is restated
  single_gather_dense      score / joint (j,k) softmax / value aggregation and the
                           five analytic gradients of one Q-anchored gather
                           (tests/test_single_gather.py:52-66; gradient algebra of
                           cuda/backward.cu:319-351 with one softmax kept).
  single_gather_banded     the same operator for a causal window, evaluated per
                           query chunk against the (chunk + w - 1) keys it can see
                           (streamed oracle of benchmarks/bench_single_gather.py:229-284).
  hypergraph_dense         the three anchored softmaxes, gather and scatter outputs
                           (cpp/torch_reference.cpp:31-54) with the pair-visibility
                           mask rule (cuda/forward.cu:33-46, tests/test_tc_paths.py:218-238).
  window_mask / gates      att3ntion/_single_gather.py:22-25; tolerances of
                           tests/test_single_gather.py:26-30 and 93-112.
"""
from __future__ import annotations

import math

import torch

NEG_INF = -1e30  # cuda/common.cuh:24

# (rel-L2, max-err / max(1, max|ref|)) gates of tests/test_single_gather.py:26-30
TOL = {
    "Y": (0.03, 0.05), "dVr": (0.04, 0.05), "dVs": (0.04, 0.05),
    "dQ": (0.06, 0.10), "dR": (0.06, 0.10), "dS": (0.06, 0.10),
}
LSE_MAX = 0.02


def window_mask(n: int, window: int, device="cpu") -> torch.Tensor:
    """[n,n] bool, query i sees key j iff i - window < j <= i (att3ntion/_single_gather.py:22-25)."""
    i = torch.arange(n, device=device)
    return (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - window)


def expand_kv(t: torch.Tensor, hq: int) -> torch.Tensor:
    """[B,Hkv,N,D] -> [B,Hq,N,D]; query head h reads KV head h // (Hq/Hkv)
    (benchmarks/bench_single_gather.py:229-284)."""
    hkv = t.shape[1]
    return t if hkv == hq else t.repeat_interleave(hq // hkv, dim=1)


def reduce_kv(g: torch.Tensor, hkv: int) -> torch.Tensor:
    """Sum a per-query-head gradient [B,Hq,N,D] back to [B,Hkv,N,D]."""
    b, hq, n, d = g.shape
    return g if hkv == hq else g.reshape(b, hkv, hq // hkv, n, d).sum(2)


def single_gather_dense(Q, R, S, Vr, Vs, mask=None, dY=None, mask_s=None):
    """One joint softmax over (j,k) per query i.

    Q [B,Hq,N,D]; R,S,Vr,Vs [B,Hkv,N,D]; mask [B,N,N] bool or None.  mask_s, if given, is the
    visibility of the S / Vs key axis and `mask` that of the R / Vr axis only (independent windows per
    axis; the reference's operator has one mask for both, tests/test_single_gather.py:52-66).
    Returns dict with Y, lse (-inf on dead rows), m, l and, if dY is given, the five
    gradients (KV gradients reduced to Hkv heads).  FP64 throughout.
    """
    Q = Q.double()
    hq, hkv = Q.shape[1], R.shape[1]
    Re, Se, Vre, Vse = (expand_kv(t.double(), hq) for t in (R, S, Vr, Vs))
    D = Q.shape[-1]
    scale = 1.0 / math.sqrt(D)
    x = torch.einsum("bhid,bhjd,bhkd->bhijk", Q, Re, Se) * scale
    if mask is not None:
        vis = (mask[:, :, :, None] & (mask if mask_s is None else mask_s)[:, :, None, :])[:, None]
        x = x.masked_fill(~vis, float("-inf"))
    flat = x.flatten(3)
    m = flat.max(-1).values
    dead = torch.isinf(m) & (m < 0)
    m_safe = torch.where(dead, torch.zeros_like(m), m)
    e = torch.exp(flat - m_safe[..., None])
    e = torch.where(dead[..., None], torch.zeros_like(e), e)
    l = e.sum(-1)
    P = (e / l.clamp_min(1e-300)[..., None]).reshape(x.shape)
    lse = torch.where(dead, torch.full_like(m, float("-inf")), m_safe + torch.log(l.clamp_min(1e-300)))
    U = torch.einsum("bhijk,bhkd->bhijd", P, Vse)                 # U[i,j,d] = sum_k P Vs
    Y = torch.einsum("bhijd,bhjd->bhid", U, Vre)
    out = {"Y": Y, "lse": lse, "m": torch.where(dead, torch.full_like(m, NEG_INF), m), "l": l}
    if dY is None:
        return out
    dY = dY.double()
    delta = (dY * Y).sum(-1)                                       # delta_i = sum_d dY.Y
    G = torch.einsum("bhid,bhjd->bhijd", dY, Vre)                  # G[i,j,d] = dY_i o Vr_j
    dP = torch.einsum("bhijd,bhkd->bhijk", G, Vse)
    gA = P * (dP - delta[..., None, None])
    Ug = torch.einsum("bhijk,bhkd->bhijd", gA, Se)
    out["dQ"] = scale * torch.einsum("bhijd,bhjd->bhid", Ug, Re)
    out["dR"] = reduce_kv(scale * torch.einsum("bhijd,bhid->bhjd", Ug, Q), hkv)
    out["dVr"] = reduce_kv(torch.einsum("bhijd,bhid->bhjd", U, dY), hkv)
    QR = torch.einsum("bhid,bhjd->bhijd", Q, Re)
    out["dS"] = reduce_kv(scale * torch.einsum("bhijk,bhijd->bhkd", gA, QR), hkv)
    out["dVs"] = reduce_kv(torch.einsum("bhijk,bhijd->bhkd", P, G), hkv)
    return out


def single_gather_banded(Q, R, S, Vr, Vs, window, dY=None, mask=None, chunk=64, q_begin=0, dtype=torch.float64):
    """Causal-window single gather without the dense cube: for each chunk of
    queries [q0,q1) only keys [q0-window+1, q1) are touched.  `mask` ([B,N,N] bool)
    may remove further keys.  Same outputs as single_gather_dense; rows < q_begin
    of Y/lse/dQ are left zero / -inf."""
    B, hq, N, D = Q.shape
    hkv = R.shape[1]
    Qd = Q.to(dtype)
    Re, Se, Vre, Vse = (expand_kv(t.to(dtype), hq) for t in (R, S, Vr, Vs))
    out = {
        "Y": torch.zeros(B, hq, N, D, dtype=dtype),
        "lse": torch.full((B, hq, N), float("-inf"), dtype=dtype),
        "m": torch.full((B, hq, N), NEG_INF, dtype=dtype),
        "l": torch.zeros(B, hq, N, dtype=dtype),
    }
    if dY is not None:
        dYd = dY.to(dtype)
        out["dQ"] = torch.zeros_like(Qd)
        acc = {n: torch.zeros_like(Re) for n in ("dR", "dS", "dVr", "dVs")}
    for q0 in range(q_begin, N, chunk):
        q1 = min(q0 + chunk, N)
        k0 = max(q0 - window + 1, 0)
        sub = window_mask(N, window)[q0:q1, k0:q1][None].expand(B, -1, -1)
        if mask is not None:
            sub = sub & mask[:, q0:q1, k0:q1]
        # pad the chunk's queries into a square problem over keys [k0,q1)
        r = _chunk_dense(Qd[:, :, q0:q1], Re[:, :, k0:q1], Se[:, :, k0:q1], Vre[:, :, k0:q1],
                         Vse[:, :, k0:q1], sub, None if dY is None else dYd[:, :, q0:q1])
        for n in ("Y", "lse", "m", "l"):
            out[n][:, :, q0:q1] = r[n]
        if dY is not None:
            out["dQ"][:, :, q0:q1] = r["dQ"]
            for n in acc:
                acc[n][:, :, k0:q1] += r[n]
    if dY is not None:
        for n in acc:
            out[n] = reduce_kv(acc[n], hkv)
    return out


def _chunk_dense(Q, R, S, Vr, Vs, vis, dY):
    """Queries [B,H,nq,D] against keys [B,H,nk,D] with visibility vis [B,nq,nk]."""
    D = Q.shape[-1]
    scale = 1.0 / math.sqrt(D)
    x = torch.einsum("bhid,bhjd,bhkd->bhijk", Q, R, S) * scale
    pair = (vis[:, :, :, None] & vis[:, :, None, :])[:, None]
    x = x.masked_fill(~pair, float("-inf"))
    flat = x.flatten(3)
    m = flat.max(-1).values
    dead = torch.isinf(m) & (m < 0)
    m_safe = torch.where(dead, torch.zeros_like(m), m)
    e = torch.where(dead[..., None], torch.zeros_like(flat), torch.exp(flat - m_safe[..., None]))
    l = e.sum(-1)
    P = (e / l.clamp_min(1e-300)[..., None]).reshape(x.shape)
    U = torch.einsum("bhijk,bhkd->bhijd", P, Vs)
    Y = torch.einsum("bhijd,bhjd->bhid", U, Vr)
    out = {"Y": Y, "l": l,
           "lse": torch.where(dead, torch.full_like(m, float("-inf")), m_safe + torch.log(l.clamp_min(1e-300))),
           "m": torch.where(dead, torch.full_like(m, NEG_INF), m)}
    if dY is None:
        return out
    delta = (dY * Y).sum(-1)
    G = torch.einsum("bhid,bhjd->bhijd", dY, Vr)
    dP = torch.einsum("bhijd,bhkd->bhijk", G, Vs)
    gA = P * (dP - delta[..., None, None])
    Ug = torch.einsum("bhijk,bhkd->bhijd", gA, S)
    out["dQ"] = scale * torch.einsum("bhijd,bhjd->bhid", Ug, R)
    out["dR"] = scale * torch.einsum("bhijd,bhid->bhjd", Ug, Q)
    out["dVr"] = torch.einsum("bhijd,bhid->bhjd", U, dY)
    out["dS"] = scale * torch.einsum("bhijk,bhid,bhjd->bhkd", gA, Q, R)
    out["dVs"] = torch.einsum("bhijk,bhijd->bhkd", P, G)
    return out


def hypergraph_dense(Q, R, S, Vq1, Vq2, Vr1, Vr2, Vs1, Vs2, mask=None, gather_mode=0, scatter=True,
                     dtype=torch.float64, valid=None):
    """Three anchored softmaxes of the same score cube (cpp/torch_reference.cpp:31-54).

    mask [B,N,N] bool: a cell of anchor a is live iff both non-anchor indices are
    visible from a (tests/test_tc_paths.py:218-238).  A fully masked anchor yields
    zeros.  Returns (Y_q, Y_r, Y_s, Y_q_, Y_r_, Y_s_) and the three LSE tensors.
    Differentiable: callers obtain the nine gradients with torch.autograd.

    The three axes may have different lengths I, J, K (no mask then, cuda/forward.cu:1281-1296).
    valid = (I_valid, J_valid, K_valid): entries of an axis at or past its valid length are padding
    that stays out of every softmax in which the axis is a key axis (cuda/forward.cu:1300-1302, 1446-1452).
    """
    Q, R, S, Vq1, Vq2, Vr1, Vr2, Vs1, Vs2 = (t.to(dtype) for t in (Q, R, S, Vq1, Vq2, Vr1, Vr2, Vs1, Vs2))
    D = Q.shape[-1]
    x = torch.einsum("bhid,bhjd,bhkd->bhijk", Q, R, S) / math.sqrt(D)

    lens = (Q.shape[2], R.shape[2], S.shape[2])
    live = [torch.arange(n, device=Q.device) < (n if valid is None or not (0 < valid[a] <= n) else valid[a])
            for a, n in enumerate(lens)]

    def anchored(xp, u_axis, v_axis):
        # xp: [b,h,anchor,u,v]; mask[b,anchor,u] & mask[b,anchor,v]; u, v below their axes' valid lengths
        if mask is not None:
            vp = (mask[:, :, :, None] & mask[:, :, None, :]).unsqueeze(1)
            xp = xp.masked_fill(~vp, float("-inf"))
        if valid is not None:
            vp = live[u_axis][:, None] & live[v_axis][None, :]
            xp = xp.masked_fill(~vp, float("-inf"))
        flat = xp.flatten(3)
        lse = torch.logsumexp(flat, -1)
        p = torch.nan_to_num(torch.softmax(flat, -1), nan=0.0).reshape(xp.shape)
        return p, lse

    Aq, lse_q = anchored(x, 1, 2)                              # [i,j,k]
    Y_q = torch.einsum("bhijk,bhjd,bhkd->bhid", Aq, Vr1, Vs1)
    zq, zr, zs = torch.zeros_like(Q), torch.zeros_like(R), torch.zeros_like(S)
    if gather_mode == 1:
        return (Y_q, zr, zs, zq, zr, zs), (lse_q, None, None)
    Ar_p, lse_r = anchored(x.permute(0, 1, 3, 2, 4), 0, 2)     # [j,i,k]
    As_p, lse_s = anchored(x.permute(0, 1, 4, 2, 3), 0, 1)     # [k,i,j]
    Ar = Ar_p.permute(0, 1, 3, 2, 4)
    As = As_p.permute(0, 1, 3, 4, 2)
    Y_r = torch.einsum("bhijk,bhid,bhkd->bhjd", Ar, Vq1, Vs1)
    Y_s = torch.einsum("bhijk,bhid,bhjd->bhkd", As, Vq1, Vr1)
    if scatter:
        Y_q_ = torch.einsum("bhijk,bhjd,bhkd->bhid", Ar * As, Vr2, Vs2)
        Y_r_ = torch.einsum("bhijk,bhid,bhkd->bhjd", Aq * As, Vq2, Vs2)
        Y_s_ = torch.einsum("bhijk,bhid,bhjd->bhkd", Aq * Ar, Vq2, Vr2)
    else:
        Y_q_, Y_r_, Y_s_ = zq, zr, zs
    return (Y_q, Y_r, Y_s, Y_q_, Y_r_, Y_s_), (lse_q, lse_r, lse_s)


def hypergraph_grads(inputs, cotangents, mask=None, gather_mode=0, scatter=True, valid=None):
    """Nine input gradients of hypergraph_dense under the six cotangents, by FP64 autograd."""
    leaves = [t.detach().double().requires_grad_(True) for t in inputs]
    outs, _ = hypergraph_dense(*leaves, mask=mask, gather_mode=gather_mode, scatter=scatter, valid=valid)
    total = None
    for o, g in zip(outs, cotangents):
        if g is None or not o.requires_grad:
            continue
        term = (o * g.double()).sum()
        total = term if total is None else total + term
    grads = torch.autograd.grad(total, leaves, allow_unused=True)
    return [torch.zeros_like(l) if g is None else g for g, l in zip(grads, leaves)]


# --------------------------------------------------------------------------- gates

def errors(actual: torch.Tensor, ref: torch.Tensor):
    """(rel-L2, max-err / max(1, max|ref|)) as in tests/test_single_gather.py:82-86."""
    a, r = actual.double().cpu(), ref.double().cpu()
    rel = (a - r).norm() / max(r.norm().item(), 1e-12)
    mx = (a - r).abs().max() / max(1.0, r.abs().max().item())
    return rel.item(), mx.item()


def check_gate(name: str, actual: torch.Tensor, ref: torch.Tensor, per_head: bool = True) -> None:
    """Global and per-(b,h) tolerance gate of tests/test_single_gather.py:89-107."""
    assert torch.isfinite(actual).all(), f"{name}: non-finite"
    if ref.abs().max().item() == 0.0:
        assert actual.abs().max().item() <= 1e-6, f"{name}: nonzero vs identically-zero ref"
        return
    rtol, mtol = TOL[name]
    rel, mx = errors(actual, ref)
    assert rel <= rtol and mx <= mtol, f"{name}: rel L2 {rel:.4f} (<= {rtol}), max {mx:.4f} (<= {mtol})"
    if not per_head:
        return
    for b in range(actual.size(0)):
        for h in range(actual.size(1)):
            if ref[b, h].abs().max().item() == 0.0:
                continue
            rel, mx = errors(actual[b, h], ref[b, h])
            assert rel <= rtol and mx <= mtol, f"{name}[b={b},h={h}]: rel L2 {rel:.4f}, max {mx:.4f}"


def lse_from_ml(m: torch.Tensor, l: torch.Tensor) -> torch.Tensor:
    m, l = m.double().cpu(), l.double().cpu()
    return torch.where(l > 0, m + torch.log(l.clamp_min(1e-300)), torch.full_like(m, float("-inf")))


def check_lse(m, l, lse_ref) -> None:
    """Dead-row set equality and |LSE - ref| <= 0.02 on live rows (tests/test_single_gather.py:110-121)."""
    lse = lse_from_ml(m, l)
    lse_ref = lse_ref.double().cpu()
    dead = torch.isinf(lse_ref) & (lse_ref < 0)
    assert torch.equal(dead, torch.isinf(lse) & (lse < 0)), "dead-row set differs"
    if (~dead).any():
        err = (lse[~dead] - lse_ref[~dead]).abs().max().item()
        assert err <= LSE_MAX, f"LSE max err {err:.4f}"


def slice_gate(host, got, window, b, lo, hi, mask=None, heads=None):
    """Full-size check of the windowed single gather on one slice: queries [lo, hi) of batch `b`
    against the banded FP64 oracle, as the reference gates a shape before it publishes a timing for it
    (benchmarks/bench_single_gather.py:887-961), restricted to a slice because the whole problem is out
    of the oracle's reach.

    host  (Q, R, S, Vr, Vs, dY) CPU tensors of the whole problem
    got   dict with the device results as tensors indexable like the whole problem: Y, m, l, dQ, and
          dR, dS, dVr, dVs (summed over query heads; only rows whose 128 contributing queries all lie in
          the slice are compared, i.e. keys lo .. hi-128 when the slice is longer than a window, so the
          result must come from a run over all query heads of the KV head)
    heads query heads the device run held (default: all); Y, m, l, dQ are compared for these only,
          `got` then holds them in this order

    Raises AssertionError on a failed gate; returns {name: rel-L2}.  Needs lo >= 127 or lo == 0.
    """
    Q, R, S, Vr, Vs, dY = host
    pre = min(lo, RING_ROWS - 1)
    sl = slice(lo - pre, hi)
    msk = None if mask is None else mask[b:b + 1, sl, sl]
    ref = single_gather_banded(Q[b:b + 1, :, sl], *[t[b:b + 1, :, sl] for t in (R, S, Vr, Vs)], window=window,
                               dY=dY[b:b + 1, :, sl], q_begin=pre, chunk=32, mask=msk)
    hs = list(range(Q.shape[1])) if heads is None else list(heads)
    rels = {}

    def gate(name, a, r):
        check_gate(name, a.float().cpu(), r)
        rels[name] = errors(a, r)[0]

    gate("Y", got["Y"][b:b + 1, :, lo:hi], ref["Y"][:, hs, pre:])
    check_lse(got["m"][b:b + 1, :, lo:hi], got["l"][b:b + 1, :, lo:hi], ref["lse"][:, hs, pre:])
    gate("dQ", got["dQ"][b:b + 1, :, lo:hi], ref["dQ"][:, hs, pre:])
    nk = hi - lo - (RING_ROWS - 1)
    if nk > 0 and all(k in got for k in ("dR", "dS", "dVr", "dVs")):
        for name in ("dR", "dS", "dVr", "dVs"):
            gate(name, got[name][b:b + 1, :, lo:lo + nk], ref[name][:, :, pre:pre + nk])
    return rels


RING_ROWS = 128   # keys a query can see at most (the kernels' resident ring); a key collects from 128 queries
