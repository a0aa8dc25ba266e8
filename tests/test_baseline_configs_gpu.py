"""The five benchmark configurations at their stated shapes and seeds, each gated against the
CPU oracle (or the reference-made golden vector) on the GPU:

  C1  three-gather, B2 N64 d_model 64 H4 (D 16), seed 0: through the projections, forward y and the
      gradients of x and of all six projection weights against the output of the reference's CPU
      naive module (tests/golden/naive_c1.pt)
  C2  three-gather, B8 N256 d_model 256 H4 (D 64), seed 1, x ~ N(0,1), Xavier-uniform weights: two
      (batch, head) pairs against the dense FP64 three-gather oracle at operator level
  C3  single gather, B4 H8 N2048 D64 w128, seed 2: two (batch, head) pairs, 192-query slice
  C4  shared KV, B4 Hq8 N8192 D128, seed 3, windows 16 / 32 / 64 (window 128 is in
      test_single_gather_gpu.py::test_full_size_properties_c4_shape): 192-query slice, repeat equality
  C5  shared KV, B1 Hq8 N131072 D128 w128, seed 4, on one GPU: a slice in the middle, and the rows
      around 16384 (a shard boundary of the 8-GPU split) computed once as part of the whole sequence
      and once from a shard that starts 128 rows earlier (q_begin): bit-identical Y, dQ

Tolerances are the reference's (tests/test_single_gather.py:26-30, tests/test_kernel_correctness.py:303-361)."""
import math

import pytest
import torch

from conftest import load_golden
from oracle import triplet_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ck():
    from att3ntion_b200 import _cuda_kernels
    return _cuda_kernels


def draw_shared(B, Hq, N, D, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    s = 1.0 / math.sqrt(D)
    Q = (torch.randn(B, Hq, N, D, generator=g) * s).to(torch.bfloat16)
    kv = [(torch.randn(B, 1, N, D, generator=g) * s).to(torch.bfloat16) for _ in range(4)]
    dY = torch.randn(B, Hq, N, D, generator=g).to(torch.bfloat16)
    return (Q, *kv, dY)


def run(ck, host, w, q_begin=0):
    Q, R, S, Vr, Vs, dY = (t.cuda() for t in host)
    Y, m, l = ck.sg_forward_raw(Q, R, S, Vr, Vs, None, w, q_begin)
    g = ck.sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, None, w, q_begin)
    ck.device_status()
    return {"Y": Y, "m": m, "l": l, "dQ": g[0], "dR": g[1], "dS": g[2], "dVr": g[3], "dVs": g[4]}


# --------------------------------------------------------------------------- C4, windows 16 / 32 / 64

@pytest.mark.parametrize("window", [16, 32, 64])
def test_c4_shape_small_windows(ck, window):
    host = draw_shared(4, 8, 8192, 128, seed=3)
    got = run(ck, host, window)
    O.slice_gate(host, got, window, 2, 4000, 4192)
    O.slice_gate(host, got, window, 0, 0, 160)                       # the ramp at the start of the sequence
    again = run(ck, host, window)
    for k in got:
        assert torch.equal(got[k], again[k]), k
        assert torch.isfinite(got[k].float()).all(), k


# --------------------------------------------------------------------------- C3

def test_c3_shape_independent_heads(ck):
    B, H, N, D, w = 4, 8, 2048, 64, 128
    g = torch.Generator(device="cpu").manual_seed(2)
    xs = [(torch.randn(B, H, N, D, generator=g) / math.sqrt(D)).to(torch.bfloat16) for _ in range(5)]
    dY = torch.randn(B, H, N, D, generator=g).to(torch.bfloat16)
    q = [t.cuda() for t in xs]
    Y, m, l = ck.sg_forward_raw(*q, None, w)
    gr = ck.sg_backward_raw(dY.cuda(), *q, Y, m, l, None, w)
    ck.device_status()
    for (b, h) in ((1, 2), (3, 7)):
        sel = lambda t: t[b:b + 1, h:h + 1]
        got = {"Y": sel(Y), "m": m[b:b + 1, h:h + 1], "l": l[b:b + 1, h:h + 1], "dQ": sel(gr[0]),
               "dR": sel(gr[1]), "dS": sel(gr[2]), "dVr": sel(gr[3]), "dVs": sel(gr[4])}
        O.slice_gate(tuple(sel(t) for t in (*xs, dY)), got, w, 0, 1024 - 96, 1024 + 96)
        O.slice_gate(tuple(sel(t) for t in (*xs, dY)), got, w, 0, 0, 160)
    again = ck.sg_backward_raw(dY.cuda(), *q, Y, m, l, None, w)
    assert all(torch.equal(a, b) for a, b in zip(gr, again))


# --------------------------------------------------------------------------- C5 on one GPU

def test_c5_shape_long_sequence_and_shard_boundary(ck):
    N, w, cut = 131072, 128, 16384
    host = draw_shared(1, 8, N, 128, seed=4)
    got = run(ck, host, w)
    O.slice_gate(host, got, w, 0, 65536 - 96, 65536 + 96)            # the middle of the sequence
    O.slice_gate(host, got, w, 0, cut - 96, cut + 96)                # straddling a shard boundary
    # the shard [cut, 2 cut) as rank 1 of an 8-way split would run it: 128 halo rows in front, q_begin = 128
    lo, hi = cut - 128, 2 * cut
    shard = tuple(t[:, :, lo:hi].contiguous() for t in host)
    part = run(ck, shard, w, q_begin=128)
    assert torch.equal(part["Y"][:, :, 128:], got["Y"][:, :, cut:hi])
    assert torch.equal(part["m"][:, :, 128:], got["m"][:, :, cut:hi])
    assert torch.equal(part["l"][:, :, 128:], got["l"][:, :, cut:hi])
    assert torch.equal(part["dQ"][:, :, 128:], got["dQ"][:, :, cut:hi])
    # key gradients: rows whose 128 contributing queries all lie inside the shard are complete there; the two
    # runs cut their query blocks in different places, so the FP32 partial sums are added in another order
    for k in ("dR", "dS", "dVr", "dVs"):
        rel, mx = O.errors(part[k][:, :, 128:hi - lo - 127], got[k][:, :, cut:hi - 127].float())
        assert rel < 0.01 and mx < 0.02, (k, rel, mx)


# --------------------------------------------------------------------------- C2 and C1 (three-gather, through the projections)

def _xavier_projections(d_model, seed):
    """Six bias-free projection weights [d_model, d_model], Xavier-uniform from `seed` (Wq, Wr, Ws, Wv_q, Wv_r, Wv_s)."""
    torch.manual_seed(seed)
    ws = []
    for _ in range(6):
        w = torch.empty(d_model, d_model)
        torch.nn.init.xavier_uniform_(w)
        ws.append(w)
    return ws


def _heads(t, H):
    b, n, dm = t.shape
    return t.reshape(b, n, H, dm // H).permute(0, 2, 1, 3)


def test_c2_shape_three_gather_operator():
    from att3ntion_b200._autograd import _HypergraphAttentionAutograd
    B, N, dm, H = 8, 256, 256, 4
    ws = _xavier_projections(dm, seed=1)
    g = torch.Generator(device="cpu").manual_seed(1)
    x = torch.randn(B, N, dm, generator=g)
    cot = [torch.randn(B, H, N, dm // H, generator=g).to(torch.bfloat16) for _ in range(3)]
    proj = [_heads(x @ w.T, H).to(torch.bfloat16) for w in ws]           # Q, R, S, Vq, Vr, Vs as the kernels see them
    Q, R, S, Vq, Vr, Vs = proj
    z = torch.zeros_like(Q)
    leaves = [t.cuda().float().requires_grad_(True) for t in (Q, R, S, Vq, z, Vr, z, Vs, z)]
    outs = _HypergraphAttentionAutograd.apply(*leaves, None, 0.0, False, 0)
    torch.autograd.backward(outs[:3], [c.cuda().float() for c in cot])
    for (b, h) in ((0, 0), (5, 3), (7, 1)):
        sub = [t[b:b + 1, h:h + 1] for t in (Q, R, S, Vq, z, Vr, z, Vs, z)]
        ref_out, _ = O.hypergraph_dense(*sub, scatter=False)
        ref_gr = O.hypergraph_grads(sub, [c[b:b + 1, h:h + 1] for c in cot] + [None] * 3, scatter=False)
        for k in range(3):
            a, r = outs[k][b:b + 1, h:h + 1].detach().float().cpu(), ref_out[k].float()
            assert torch.allclose(a, r, rtol=5e-2, atol=5e-2 * max(1.0, r.abs().max().item())), (k, b, h)
        for k, (rt, at) in zip((0, 1, 2, 3, 5, 7), [(5e-2, 1e-1)] * 3 + [(2e-2, 2e-2)] * 3):
            a, r = leaves[k].grad[b:b + 1, h:h + 1].float().cpu(), ref_gr[k].float()
            assert torch.allclose(a, r, rtol=rt, atol=at * max(1.0, r.abs().max().item())), (k, b, h)


def test_c1_against_the_reference_naive_module():
    """x -> six projections -> three-gather kernels (D = 16) -> gelu sum -> merged heads, with the weights and
    inputs of the golden file: y, dx and the six weight gradients against the reference's FP32 CPU naive
    module.  The kernels see BF16 operands, so the comparison is a tolerance (rel-L2), not equality."""
    from att3ntion_b200._autograd import QuickGELU, _HypergraphAttentionAutograd
    g = load_golden("naive_c1.pt")
    H = 4
    names = ["Wq", "Wr", "Ws", "Wv_q", "Wv_r", "Wv_s"]
    ws = [g["state_dict"][f"{n}.weight"].cuda().requires_grad_(True) for n in names]
    x = g["x"].cuda().requires_grad_(True)
    Q, R, S, Vq, Vr, Vs = (_heads(x @ w.T, H) for w in ws)
    z = torch.zeros_like(Q)
    Yq, Yr, Ys, *_ = _HypergraphAttentionAutograd.apply(Q, R, S, Vq, z, Vr, z, Vs, z, None, 0.0, False, 0)
    gelu = QuickGELU()
    y = (gelu(Yq) + gelu(Yr) + gelu(Ys)).permute(0, 2, 1, 3).reshape(x.shape)
    y.backward(g["dY"].cuda())
    rel = lambda a, r: ((a.detach().double().cpu() - r.double()).norm() / r.double().norm()).item()
    assert rel(y, g["y"]) < 0.03
    assert rel(x.grad, g["dx"]) < 0.06
    for n, w in zip(names, ws):
        assert rel(w.grad, g["dW"][f"{n}.weight"]) < 0.06, n
