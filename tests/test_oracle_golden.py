"""Pins the CPU oracle (oracle/triplet_oracle.py) against the golden vectors that
tests/golden/make_golden.py produced from the reference's own oracles."""
import json

import pytest
import torch

from conftest import GOLDEN, golden_files, load_golden
from oracle import triplet_oracle as O

NAMES = ["Q", "R", "S", "Vr", "Vs"]
GRADS = ["dQ", "dR", "dS", "dVr", "dVs"]


def close(a, b, tol=2e-5):
    a, b = a.double(), b.double()
    assert a.shape == b.shape
    fin = torch.isfinite(b)
    assert torch.equal(fin, torch.isfinite(a))
    scale = max(1.0, b[fin].abs().max().item()) if fin.any() else 1.0
    assert (a[fin] - b[fin]).abs().max().item() <= tol * scale


@pytest.mark.parametrize("name", golden_files("sg_"))
def test_single_gather_dense_matches_reference_oracle(name):
    g = load_golden(name)
    out = O.single_gather_dense(*[g["inputs"][n] for n in NAMES], mask=g["mask"], dY=g["dY"])
    close(out["Y"], g["Y"])
    close(out["lse"], g["lse"])
    for k in GRADS:
        close(out[k], g[k])


@pytest.mark.parametrize("name", golden_files("shared_"))
def test_shared_kv_matches_reference_oracle(name):
    g = load_golden(name)
    B, _, N, _ = g["inputs"]["Q"].shape
    mask = O.window_mask(N, g["window"])[None].expand(B, -1, -1)
    if g["extra_mask"] is not None:
        mask = mask & g["extra_mask"]
    out = O.single_gather_dense(*[g["inputs"][n] for n in NAMES], mask=mask, dY=g["dY"])
    close(out["Y"], g["Y"])
    close(out["lse"], g["lse"])
    for k in GRADS:
        close(out[k], g[k])
        if k != "dQ":
            assert out[k].shape[1] == 1
    # the banded restatement used for full-size shapes agrees with the dense one
    band = O.single_gather_banded(*[g["inputs"][n] for n in NAMES], window=g["window"], dY=g["dY"],
                                  mask=g["extra_mask"], chunk=24)
    close(band["Y"], g["Y"])
    close(band["lse"], g["lse"])
    for k in GRADS:
        close(band[k], g[k])


HG_NAMES = ["Q", "R", "S", "Vq_1", "Vq_2", "Vr_1", "Vr_2", "Vs_1", "Vs_2"]


@pytest.mark.parametrize("name", [n for n in golden_files("hg_") if "masked" not in n])
def test_hypergraph_unmasked_matches_torch_reference(name):
    g = load_golden(name)
    ins = [g["inputs"][n] for n in HG_NAMES]
    outs, _ = O.hypergraph_dense(*ins)
    for o, r in zip(outs, g["outputs"]):
        close(o, r)
    grads = O.hypergraph_grads(ins, g["cotangents"])
    for a, r in zip(grads, g["grads"]):
        close(a, r, 5e-5)


@pytest.mark.parametrize("name", golden_files("hg_masked_"))
def test_hypergraph_masked_gathers_match_reference_rule(name):
    g = load_golden(name)
    ins = [g["inputs"][n] for n in HG_NAMES]
    outs, _ = O.hypergraph_dense(*ins, mask=g["mask"], scatter=False)
    for o, r in zip(outs[:3], g["outputs"]):
        close(o, r)
    grads = O.hypergraph_grads(ins, list(g["cotangents"]) + [None] * 3, mask=g["mask"], scatter=False)
    for a, r in zip(grads, g["grads"]):
        close(a, r, 5e-5)


def test_gather_mode_one_equals_single_gather():
    g = load_golden("sg_B1H2N33D64_s1_causal.pt")
    x = g["inputs"]
    z = torch.zeros_like(x["Q"])
    outs, _ = O.hypergraph_dense(x["Q"], x["R"], x["S"], z, z, x["Vr"], z, x["Vs"], z, mask=g["mask"], gather_mode=1)
    close(outs[0], g["Y"])


def test_window_mask_and_gates():
    m = O.window_mask(6, 3)
    assert m.tolist()[4] == [False, False, True, True, True, False]
    assert O.window_mask(4, 9).equal(torch.tril(torch.ones(4, 4, dtype=torch.bool)))
    O.check_gate("Y", torch.ones(1, 1, 4, 4) * 1.01, torch.ones(1, 1, 4, 4))
    with pytest.raises(AssertionError):
        O.check_gate("Y", torch.ones(1, 1, 4, 4) * 1.2, torch.ones(1, 1, 4, 4))
    with pytest.raises(AssertionError):                  # dead-row sets must agree
        O.check_lse(torch.tensor([[0.0]]), torch.tensor([[1.0]]), torch.tensor([[float("-inf")]]))


def test_three_gather_oracle_matches_the_reference_naive_module():
    """tests/golden/naive_c1.pt holds the reference's CPU naive module (att3ntion/_naive.py:80-160,
    _HypergraphAttentionNaive with head subspaces) at B2 N64 d_model 64 H4, seed 0: its weights, input,
    output and the gradients of the input and of the six projections.  Restating its forward around the
    oracle's three-gather (projections, head split, gelu(Y_q) + gelu(Y_r) + gelu(Y_s), heads merged) must
    give the same numbers: this pins hypergraph_dense and its autograd gradients to the reference module."""
    g = load_golden("naive_c1.pt")
    H = 4
    names = ["Wq", "Wr", "Ws", "Wv_q", "Wv_r", "Wv_s"]
    ws = [g["state_dict"][f"{n}.weight"].double().requires_grad_(True) for n in names]
    x = g["x"].double().requires_grad_(True)

    def heads(t):
        b, n, dm = t.shape
        return t.reshape(b, n, H, dm // H).permute(0, 2, 1, 3)

    Q, R, S, Vq, Vr, Vs = (heads(x @ w.T) for w in ws)
    z = torch.zeros_like(Q)
    outs, _ = O.hypergraph_dense(Q, R, S, Vq, z, Vr, z, Vs, z, scatter=False)
    gelu = lambda t: t * torch.sigmoid(1.702 * t)
    y = (gelu(outs[0]) + gelu(outs[1]) + gelu(outs[2])).permute(0, 2, 1, 3).reshape(x.shape)
    y.backward(g["dY"].double())
    close(y.detach(), g["y"], 1e-4)
    close(x.grad, g["dx"], 1e-4)
    for n, w in zip(names, ws):
        close(w.grad, g["dW"][f"{n}.weight"], 1e-4)
