"""GPU parity tests of the dense anchored gather: the un-windowed single gather
(arbitrary masks, any N) and the three-gather HypergraphAttention operator, against the
golden vectors made from the reference's oracles and against the CPU oracle.

Gates: single gather as in tests/test_single_gather.py:26-30 of the reference; three-gather
outputs allclose(rtol 5e-2, atol 5e-2 * max(1, max|ref|)), gradients of Q/R/S
(5e-2, 1e-1 * ...), of the values (2e-2, 2e-2 * ...) as in tests/test_kernel_correctness.py:303-361."""
import pytest
import torch

from conftest import golden_files, load_golden
from oracle import triplet_oracle as O

pytestmark = pytest.mark.gpu

NAMES = ["Q", "R", "S", "Vr", "Vs"]
GRADS = ["dQ", "dR", "dS", "dVr", "dVs"]
HG_NAMES = ["Q", "R", "S", "Vq_1", "Vq_2", "Vr_1", "Vr_2", "Vs_1", "Vs_2"]


@pytest.fixture(scope="module")
def ck():
    from att3ntion_b200 import _cuda_kernels
    return _cuda_kernels


# --------------------------------------------------------------------------- dense single gather

DENSE_SG = [n for n in golden_files("sg_") if "_window" not in n]


@pytest.mark.parametrize("name", DENSE_SG)
def test_dense_single_gather_golden_bridge(name):
    from att3ntion_b200 import single_gather_attention
    g = load_golden(name)
    leaves = {n: g["inputs"][n].cuda().requires_grad_(True) for n in NAMES}
    mask = None if g["mask"] is None else g["mask"].cuda()
    Y = single_gather_attention(*[leaves[n] for n in NAMES], mask)
    Y.backward(g["dY"].cuda())
    O.check_gate("Y", Y.detach().float().cpu(), g["Y"])
    dead = torch.isinf(g["lse"])
    if dead.any():
        assert Y.detach().cpu()[dead].abs().max().item() == 0.0
    for gname, n in zip(GRADS, NAMES):
        O.check_gate(gname, leaves[n].grad.float().cpu(), g[gname])


@pytest.mark.parametrize("name", [n for n in DENSE_SG if "N16D" in n or "N128D" in n or "N32D" in n])
def test_dense_single_gather_golden_lowlevel(ck, name):
    g = load_golden(name)
    q = [g["inputs"][n].cuda() for n in NAMES]
    mask = None if g["mask"] is None else g["mask"].cuda().contiguous()
    Y, m, l = ck.single_gather_forward(*q, mask)
    O.check_gate("Y", Y.float().cpu(), g["Y"])
    O.check_lse(m, l, g["lse"])
    grads = ck.single_gather_backward(g["dY"].cuda(), *q, Y, m, l, mask)
    ck.device_status()
    for gname, t in zip(GRADS, grads):
        O.check_gate(gname, t.float().cpu(), g[gname])
    again = ck.single_gather_backward(g["dY"].cuda(), *q, Y, m, l, mask)
    assert all(torch.equal(a, b) for a, b in zip(grads, again)), "repeated backward must be bit-identical"


@pytest.mark.parametrize("N,D", [(144, 64), (272, 128)])
def test_dense_multi_tile_causal_and_random(ck, N, D):
    """More than one 128-key tile per side, causal and random masks (the merge across tiles)."""
    gen = torch.Generator().manual_seed(N)
    xs = {n: torch.randn(1, 2, N, D, generator=gen).to(torch.bfloat16) for n in NAMES}
    dY = torch.randn(1, 2, N, D, generator=gen).to(torch.bfloat16)
    for kind in ("causal", "random"):
        if kind == "causal":
            mask = torch.tril(torch.ones(1, N, N, dtype=torch.bool))
        else:
            mask = torch.rand(1, N, N, generator=gen) < 0.5
            mask[:, 3, :] = False
        ref = O.single_gather_dense(*[xs[n] for n in NAMES], mask=mask, dY=dY)
        q = [xs[n].cuda() for n in NAMES]
        mk = mask.cuda().contiguous()
        Y, m, l = ck.single_gather_forward(*q, mk)
        grads = ck.single_gather_backward(dY.cuda(), *q, Y, m, l, mk)
        ck.device_status()
        O.check_gate("Y", Y.float().cpu(), ref["Y"])
        O.check_lse(m, l, ref["lse"])
        for gname, t in zip(GRADS, grads):
            O.check_gate(gname, t.float().cpu(), ref[gname])


# --------------------------------------------------------------------------- three-gather

def hg_close(actual, ref, rtol, atol_scale, what):
    a, r = actual.double().cpu(), ref.double()
    atol = atol_scale * max(1.0, r.abs().max().item())
    bad = (a - r).abs() > atol + rtol * r.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())} elements off, max err {(a - r).abs().max().item():.4f} (atol {atol:.4f})"


def run_hg(ck, g, mask):
    ins = [g["inputs"][n].cuda() for n in HG_NAMES]
    # gather-only comparison: the scatter value tensors are zeroed so the scatter outputs vanish
    for k in (4, 6, 8):
        ins[k] = torch.zeros_like(ins[k])
    out = ck.forward(*ins, 0.0, -1, -1, -1, mask, 0)
    cot = [c.cuda() for c in g["cotangents"][:3]] + [torch.zeros_like(ins[0]) for _ in range(3)]
    grads = ck.backward(*cot, *ins, *out[6:12], 0.0, mask, out[0], out[1], out[2])
    ck.device_status()
    return out, grads


@pytest.mark.parametrize("name", [n for n in golden_files("hg_") if "masked" not in n])
def test_three_gather_unmasked_gathers(ck, name):
    g = load_golden(name)
    out, grads = run_hg(ck, g, None)
    for k, what in enumerate(("Y_q", "Y_r", "Y_s")):
        hg_close(out[k], g["outputs"][k], 5e-2, 5e-2, what)
        assert out[3 + k].abs().max().item() == 0.0
    # gradients of the gather-only objective from the FP64 oracle on the same inputs
    ins = [g["inputs"][n] for n in HG_NAMES]
    for k in (4, 6, 8):
        ins[k] = torch.zeros_like(ins[k])
    ref = O.hypergraph_grads(ins, list(g["cotangents"][:3]) + [None] * 3, scatter=False)
    for k, n in enumerate(HG_NAMES):
        hg_close(grads[k], ref[k], 5e-2, 1e-1 if k < 3 else 2e-2, f"d{n}")


@pytest.mark.parametrize("name", [n for n in golden_files("hg_") if "masked" not in n])
def test_three_gather_with_scatter_golden(ck, name):
    """All six outputs and the nine gradients under six cotangents, second value tensors in use,
    against the vectors made with the reference's own oracle (cpp/torch_reference.cpp:24-57)."""
    g = load_golden(name)
    ins = [g["inputs"][n].cuda() for n in HG_NAMES]
    out = ck.forward(*ins, 0.0, -1, -1, -1, None, 0)
    for k, what in enumerate(("Y_q", "Y_r", "Y_s", "Y_q_", "Y_r_", "Y_s_")):
        hg_close(out[k], g["outputs"][k], 5e-2, 5e-2, what)
    cot = [c.cuda() for c in g["cotangents"]]
    grads = ck.backward(*cot, *ins, *out[6:12], 0.0, None, out[0], out[1], out[2])
    ck.device_status()
    for k, n in enumerate(HG_NAMES):
        hg_close(grads[k], g["grads"][k], 5e-2, 1e-1 if k < 3 else 2e-2, f"d{n}")


@pytest.mark.parametrize("kind", ["causal", "dead_rows"])
def test_three_gather_scatter_masked_vs_oracle(ck, kind):
    """Scatter terms under a mask (each softmax keeps its own support), against the FP64 oracle."""
    B, H, N, D = 1, 2, 32, 64
    gen = torch.Generator().manual_seed(11)
    ins = [(torch.randn(B, H, N, D, generator=gen) * (0.6 if k < 3 else 1.0)).bfloat16() for k in range(9)]
    cot = [torch.randn(B, H, N, D, generator=gen).bfloat16() for _ in range(6)]
    mask = torch.tril(torch.ones(N, N, dtype=torch.bool)).expand(B, N, N).clone()
    if kind == "dead_rows":
        mask[:, 5, :] = False
        mask[:, :, 9] = False
    out = ck.forward(*[t.cuda() for t in ins], 0.0, -1, -1, -1, mask.cuda().contiguous(), 0)
    ref, _ = O.hypergraph_dense(*ins, mask=mask, scatter=True)
    for k, what in enumerate(("Y_q", "Y_r", "Y_s", "Y_q_", "Y_r_", "Y_s_")):
        hg_close(out[k], ref[k], 5e-2, 5e-2, what)
    grads = ck.backward(*[c.cuda() for c in cot], *[t.cuda() for t in ins], *out[6:12], 0.0,
                        mask.cuda().contiguous(), out[0], out[1], out[2])
    ck.device_status()
    gref = O.hypergraph_grads(ins, cot, mask=mask, scatter=True)
    for k, n in enumerate(HG_NAMES):
        hg_close(grads[k], gref[k], 5e-2, 1e-1 if k < 3 else 2e-2, f"d{n}")


@pytest.mark.parametrize("masked", [False, True])
def test_three_gather_scatter_two_key_tiles(ck, masked):
    """Scatter terms across more than one 128-key tile (N = 160: a full and a ragged tile on every axis),
    with and without a non-symmetric mask, against the FP64 oracle; and bit-identical on a second call
    (the tensor-core scatter path has a fixed summation order)."""
    B, H, N, D = 1, 1, 160, 64
    gen = torch.Generator().manual_seed(23)
    ins = [(torch.randn(B, H, N, D, generator=gen) * (0.5 if k < 3 else 1.0)).bfloat16() for k in range(9)]
    cot = [torch.randn(B, H, N, D, generator=gen).bfloat16() for _ in range(6)]
    mask = None
    if masked:
        mask = torch.tril(torch.ones(N, N, dtype=torch.bool)) & (torch.rand(N, N, generator=gen) < 0.8)
        mask |= torch.eye(N, dtype=torch.bool)
        mask = mask.expand(B, N, N).clone()
    dm = None if mask is None else mask.cuda().contiguous()
    dins = [t.cuda() for t in ins]
    out = ck.forward(*dins, 0.0, -1, -1, -1, dm, 0)
    ref, _ = O.hypergraph_dense(*ins, mask=mask, scatter=True)
    for k, what in enumerate(("Y_q", "Y_r", "Y_s", "Y_q_", "Y_r_", "Y_s_")):
        hg_close(out[k], ref[k], 5e-2, 5e-2, what)
    dcot = [c.cuda() for c in cot]
    grads = ck.backward(*dcot, *dins, *out[6:12], 0.0, dm, out[0], out[1], out[2])
    ck.device_status()
    gref = O.hypergraph_grads(ins, cot, mask=mask, scatter=True)
    for k, n in enumerate(HG_NAMES):
        hg_close(grads[k], gref[k], 5e-2, 1e-1 if k < 3 else 2e-2, f"d{n}")
    out2 = ck.forward(*dins, 0.0, -1, -1, -1, dm, 0)
    grads2 = ck.backward(*dcot, *dins, *out2[6:12], 0.0, dm, out2[0], out2[1], out2[2])
    assert all(torch.equal(a, b) for a, b in zip(out[:6], out2[:6]))
    assert all(torch.equal(a, b) for a, b in zip(grads, grads2))


def _axes_inputs(B, H, lens, D, seed, scatter_values=False):
    """Nine inputs with one length per axis (Q-like [I], R-like [J], S-like [K]) and six cotangents; the second value
    tensors are zero unless asked for, so that the scatter outputs vanish."""
    gen = torch.Generator().manual_seed(seed)
    I, J, K = lens
    axis = {"Q": I, "Vq_1": I, "Vq_2": I, "R": J, "Vr_1": J, "Vr_2": J, "S": K, "Vs_1": K, "Vs_2": K}
    ins = []
    for k, n in enumerate(HG_NAMES):
        t = (torch.randn(B, H, axis[n], D, generator=gen) * (0.5 if k < 3 else 1.0)).bfloat16()
        if n.endswith("_2") and not scatter_values:
            t = torch.zeros_like(t)
        ins.append(t)
    cot = [torch.randn(B, H, n, D, generator=gen).bfloat16() for n in (I, J, K)]
    cot += [torch.zeros(B, H, n, D).bfloat16() for n in (I, J, K)]
    return ins, cot


@pytest.mark.parametrize("lens,D", [((48, 160, 32), 64), ((144, 16, 272), 128), ((32, 48, 16), 16)])
def test_three_gather_unequal_axes_vs_oracle(ck, lens, D):
    """I != J != K without a mask (cuda/forward.cu:1281-1296; every output has the length of its own axis): the three
    gathers, their statistics and the nine gradients against the FP64 oracle, key axes spanning one, two and three
    128-key tiles; bit-identical on a second call."""
    B, H = 2, 2
    ins, cot = _axes_inputs(B, H, lens, D, seed=31)
    dins, dcot = [t.cuda() for t in ins], [c.cuda() for c in cot]
    out = ck.forward(*dins, 0.0, -1, -1, -1, None, 0)
    ref, lse = O.hypergraph_dense(*ins, scatter=False)
    for k, what in enumerate(("Y_q", "Y_r", "Y_s")):
        assert out[k].shape == ref[k].shape
        hg_close(out[k], ref[k], 5e-2, 5e-2, what)
        assert not out[3 + k].any()
        O.check_lse(out[6 + 2 * k].cpu(), out[7 + 2 * k].cpu(), lse[k])
    grads = ck.backward(*dcot, *dins, *out[6:12], 0.0, None, out[0], out[1], out[2])
    ck.device_status()
    gref = O.hypergraph_grads(ins, cot, scatter=False)
    for k, n in enumerate(HG_NAMES):
        assert grads[k].shape == ins[k].shape
        hg_close(grads[k], gref[k], 5e-2, 1e-1 if k < 3 else 2e-2, f"d{n}")
    out2 = ck.forward(*dins, 0.0, -1, -1, -1, None, 0)
    grads2 = ck.backward(*dcot, *dins, *out2[6:12], 0.0, None, out2[0], out2[1], out2[2])
    assert all(torch.equal(a, b) for a, b in zip(out[:3], out2[:3]))
    assert all(torch.equal(a, b) for a, b in zip(grads, grads2))


@pytest.mark.parametrize("lens,valid", [((160, 160, 160), (100, 140, 37)), ((48, 160, 32), (48, 129, 5))])
def test_three_gather_axis_valid_lengths(ck, lens, valid):
    """I_valid, J_valid, K_valid (cuda/forward.cu:1300-1302, 1446-1452): entries of an axis past its valid length stay
    out of every softmax in which that axis is a key axis; all anchors are still computed.  Forward against the
    oracle, and unchanged when the padded entries are overwritten."""
    B, H, D = 1, 2, 64
    ins, _ = _axes_inputs(B, H, lens, D, seed=37)
    dins = [t.cuda() for t in ins]
    out = ck.forward(*dins, 0.0, *valid, None, 0)
    ck.device_status()
    ref, lse = O.hypergraph_dense(*ins, scatter=False, valid=valid)
    for k, what in enumerate(("Y_q", "Y_r", "Y_s")):
        hg_close(out[k], ref[k], 5e-2, 5e-2, what)
        O.check_lse(out[6 + 2 * k].cpu(), out[7 + 2 * k].cpu(), lse[k])
    # the padded key rows are never read as keys: Y_q depends on R, Vr_1 below J_valid and S, Vs_1 below K_valid only
    poked = [t.clone() for t in dins]
    for idx, axis in ((1, 1), (5, 1), (2, 2), (7, 2)):
        poked[idx][:, :, valid[axis]:] = 3.0
    out_p = ck.forward(*poked, 0.0, *valid, None, 0)
    assert torch.equal(out[0], out_p[0]) and torch.equal(out[6], out_p[6]) and torch.equal(out[7], out_p[7])


def test_three_gather_axes_rejections(ck):
    """A mask and the scatter outputs need I == J == K, as in the reference (cuda/forward.cu:1292, 1545)."""
    B, H, D = 1, 1, 64
    ins, _ = _axes_inputs(B, H, (32, 48, 32), D, seed=41)
    dins = [t.cuda() for t in ins]
    mask = torch.ones(B, 32, 32, dtype=torch.bool, device="cuda")
    with pytest.raises(RuntimeError, match="equal shapes"):
        ck.forward(*dins, 0.0, -1, -1, -1, mask, 0)
    ins2, _ = _axes_inputs(B, H, (32, 48, 32), D, seed=41, scatter_values=True)
    with pytest.raises(RuntimeError, match="Scatter requires I == J == K"):
        ck.forward(*[t.cuda() for t in ins2], 0.0, -1, -1, -1, None, 0)
    bad = list(dins)
    bad[3] = bad[3][:, :, :16].contiguous()          # Vq_1 shorter than Q
    with pytest.raises(RuntimeError, match="Vq_1"):
        ck.forward(*bad, 0.0, -1, -1, -1, None, 0)


@pytest.mark.parametrize("name", golden_files("hg_masked_"))
def test_three_gather_masked(ck, name):
    g = load_golden(name)
    out, grads = run_hg(ck, g, g["mask"].cuda().contiguous())
    for k, what in enumerate(("Y_q", "Y_r", "Y_s")):
        hg_close(out[k], g["outputs"][k], 5e-2, 5e-2, what)
    for k, n in enumerate(HG_NAMES):
        hg_close(grads[k], g["grads"][k], 5e-2, 1e-1 if k < 3 else 2e-2, f"d{n}")
    # fully masked anchors: Y = 0 and (m, l) = (-1e30, 0)
    dead = ~g["mask"].any(-1)                               # [B, N]
    if dead.any():
        idx = dead[:, None, :].expand(-1, out[0].shape[1], -1)
        assert out[0].cpu()[idx].abs().max().item() == 0.0
        assert (out[6].cpu()[idx] == -1e30).all() and (out[7].cpu()[idx] == 0).all()


def test_gather_mode_one_matches_single_gather(ck):
    g = load_golden("sg_B1H2N16D64_s0_none.pt")
    x = {n: g["inputs"][n].cuda() for n in NAMES}
    z = torch.zeros_like(x["Q"])
    out = ck.forward(x["Q"], x["R"], x["S"], z, z, x["Vr"], z, x["Vs"], z, 0.0, -1, -1, -1, None, 1)
    O.check_gate("Y", out[0].float().cpu(), g["Y"])
    assert out[1].abs().max().item() == 0.0 and out[2].abs().max().item() == 0.0
    assert (out[8] > 1e29).all() and (out[9] == 1).all()      # statistics that null the other softmaxes


def test_module_forward_backward_and_compile():
    """HypergraphAttention end to end (projections by cuBLAS, the op by the kernels), against the
    module-level FP64 restatement built from the oracle; then the same module under torch.compile."""
    from att3ntion_b200 import HypergraphAttention
    torch.manual_seed(0)
    mod = HypergraphAttention(64, 4).cuda()
    x = torch.randn(2, 40, 64, device="cuda", requires_grad=True)
    y = mod(x)
    y.square().mean().backward()
    assert torch.isfinite(y).all() and torch.isfinite(x.grad).all()

    xd = x.detach().double().cpu().requires_grad_(True)
    w = {k: v.detach().double().cpu() for k, v in mod.state_dict().items()}
    heads = lambda t: t.reshape(2, 40, 4, 16).permute(0, 2, 1, 3)
    lin = lambda name, bias: xd @ w[f"{name}.weight"].T + (w[f"{name}.bias"] if bias else 0)
    Q, R, S = heads(lin("Wq", False)), heads(lin("Wr", False)), heads(lin("Ws", False))
    Vq, Vr, Vs = heads(lin("Wv_q", True)), heads(lin("Wv_r", True)), heads(lin("Wv_s", True))
    z = torch.zeros_like(Vq)
    (Yq, Yr, Ys, *_), _ = O.hypergraph_dense(Q, R, S, Vq, z, Vr, z, Vs, z, scatter=False)
    gelu = lambda t: t * torch.sigmoid(1.702 * t)
    yr = (gelu(Yq) + gelu(Yr) + gelu(Ys)).permute(0, 2, 1, 3).reshape(2, 40, 64) @ w["Wo.weight"].T + w["Wo.bias"]
    yr.square().mean().backward()
    rel = (y.detach().double().cpu() - yr.detach()).norm() / yr.detach().norm()
    relg = (x.grad.double().cpu() - xd.grad).norm() / xd.grad.norm()
    assert rel < 0.03 and relg < 0.06, (rel.item(), relg.item())

    compiled = torch.compile(mod)
    yc = compiled(x.detach())
    assert torch.allclose(yc, y.detach(), atol=1e-2, rtol=1e-2)


def test_module_single_gather_window_route():
    from att3ntion_b200 import HypergraphAttention
    torch.manual_seed(1)
    mod = HypergraphAttention(128, 2, gather_mode=1, window=16).cuda()
    x = torch.randn(1, 50, 128, device="cuda", requires_grad=True)
    y = mod(x)
    y.sum().backward()
    assert y.shape == (1, 50, 128) and torch.isfinite(y).all() and torch.isfinite(x.grad).all()
    assert mod.Wv_q is None
    with pytest.raises(ValueError):
        HypergraphAttention(64, 4, scatter=True, gather_mode=1)
    with pytest.raises(ValueError):
        HypergraphAttention(64, 4, window=8)


def test_module_with_scatter_terms():
    """HypergraphAttention(scatter=True): the six-output operator end to end through autograd."""
    from att3ntion_b200 import HypergraphAttention
    torch.manual_seed(2)
    mod = HypergraphAttention(64, 2, scatter=True).cuda()
    x = torch.randn(2, 32, 64, device="cuda", requires_grad=True)
    y = mod(x)
    y.square().mean().backward()
    assert y.shape == x.shape and torch.isfinite(y).all() and torch.isfinite(x.grad).all()
    assert all(torch.isfinite(p.grad).all() for p in mod.parameters() if p.grad is not None)
    assert mod.Wv_q.weight.grad.abs().max().item() > 0
