"""Generates the golden vectors under tests/golden/ from the REFERENCE's own oracles.

Run in a container that has the reference mounted:

    python tests/golden/make_golden.py [--reference <path of the reference checkout>]

What is imported from the reference (never copied):
  * tests/test_single_gather.py::reference      fp64 single-gather oracle (52-66)
  * tests/test_tc_paths.py::_ref_gather_masked  masked three-gather rule (218-238)
  * cpp/torch_reference.cpp                     three gathers + three scatters,
                                                JIT-built into oracle/_ref/ (24-57)
  * att3ntion/_naive.py::_HypergraphAttentionNaive   module-level CPU naive path
  * cuda/common.cuh sg_row_bounds/sg_col_bounds/sg_pack_mask32 through the small
    driver oracle/ref_bounds_dump.cpp, compiled in place into oracle/_ref/

The reference test modules import the compiled CUDA extension and skip without a
GPU, so they are loaded with an empty stand-in for ``att3ntion._cuda_kernels``
and with ``torch.cuda.is_available`` answering True for the duration of the
import; only pure-torch functions are then called, on the CPU.

Outputs (small .pt files, inputs stored as BF16, results as FP32):
  sg_*.pt      single gather, independent heads     Y, lse, dQ,dR,dS,dVr,dVs
  shared_*.pt  single gather, one shared KV head    same, KV grads [B,1,N,D]
  hg_*.pt      three-gather                         six outputs + nine grads
  naive_c1.pt  _HypergraphAttentionNaive at B2 N64 d_model64 H4, seed 0
  bounds.json  tile ranges and packed mask words
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import math
import os
import subprocess
import sys
import types
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
NAMES = ["Q", "R", "S", "Vr", "Vs"]


def load_reference_modules(ref: Path, torch_kernels):
    sys.modules.setdefault("att3ntion._cuda_kernels", types.ModuleType("att3ntion._cuda_kernels"))
    sys.modules.setdefault("att3ntion._torch_kernels", torch_kernels)   # the JIT-built cpp/torch_reference.cpp
    sys.path.insert(0, str(ref))
    sys.path.insert(0, str(ref / "tests"))
    real = torch.cuda.is_available
    torch.cuda.is_available = lambda: True
    try:
        mods = {}
        for name in ("test_single_gather", "test_tc_paths"):
            spec = importlib.util.spec_from_file_location(name, ref / "tests" / f"{name}.py")
            mod = importlib.util.module_from_spec(spec)
            sys.modules[name] = mod
            spec.loader.exec_module(mod)
            mods[name] = mod
    finally:
        torch.cuda.is_available = real
    import att3ntion._naive as naive
    mods["naive"] = naive
    return mods


def draw(shape_q, shape_kv, seed, scale):
    g = torch.Generator(device="cpu").manual_seed(seed)
    xs = {"Q": (torch.randn(*shape_q, generator=g) * scale).to(torch.bfloat16)}
    for n in NAMES[1:]:
        xs[n] = (torch.randn(*shape_kv, generator=g) * scale).to(torch.bfloat16)
    dY = (torch.randn(*shape_q, generator=g) * scale).to(torch.bfloat16)
    return xs, dY


def make_mask(kind, B, N, seed):
    i = torch.arange(N)
    if kind == "none":
        return None
    if kind == "causal":
        m = i[None, :] <= i[:, None]
    elif kind.startswith("window"):
        w = int(kind[6:])
        m = (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - w)
    elif kind == "random_dead":
        g = torch.Generator().manual_seed(seed)
        m = torch.rand(B, N, N, generator=g) < 0.6
        m[:, N // 2, :] = False
        return m
    elif kind.startswith("windowholes"):
        raise ValueError(kind)
    else:
        raise ValueError(kind)
    return m[None].expand(B, -1, -1).contiguous()


def single_gather_cases(tsg):
    cases = [  # B, H, N, D, seed, scale, mask kind
        (1, 2, 16, 64, 0, 1.0, "none"), (1, 2, 33, 64, 1, 0.5, "causal"), (1, 2, 65, 128, 2, 1.0, "window16"),
        (1, 2, 33, 128, 0, 1.0, "random_dead"), (2, 1, 32, 128, 0, 1.0, "random_dead"),
        (1, 1, 128, 64, 0, 1.0, "none"), (1, 1, 128, 128, 0, 1.0, "window16"), (1, 2, 65, 64, 1, 1.0, "causal"),
        (1, 2, 160, 128, 3, 1.0, "window128"), (2, 2, 96, 64, 4, 1.0, "window32"),
    ]
    for B, H, N, D, seed, scale, kind in cases:
        xs, dY = draw((B, H, N, D), (B, H, N, D), seed, scale)
        mask = make_mask(kind, B, N, seed)
        leaves = {n: xs[n].double().requires_grad_(True) for n in NAMES}
        Y, lse = tsg.reference(*[leaves[n] for n in NAMES], mask)
        Y.backward(dY.double())
        out = {"inputs": xs, "dY": dY, "mask": mask, "kind": kind, "Y": Y.detach().float(), "lse": lse.detach().float()}
        for g, n in zip(["dQ", "dR", "dS", "dVr", "dVs"], NAMES):
            out[g] = leaves[n].grad.float()
        torch.save(out, HERE / f"sg_B{B}H{H}N{N}D{D}_s{seed}_{kind}.pt")


def shared_cases(tsg):
    cases = [  # B, Hq, N, seed, window, extra-mask
        (1, 8, 32, 7, 32, False), (1, 8, 65, 11, 32, False), (2, 8, 33, 7, 32, False), (1, 4, 129, 5, 128, False),
        (1, 4, 65, 6, 16, False), (1, 4, 144, 8, 64, True), (1, 3, 48, 9, 128, False),
    ]
    D = 128
    for B, Hq, N, seed, w, holes in cases:
        xs, dY = draw((B, Hq, N, D), (B, 1, N, D), seed, 1.0)
        i = torch.arange(N)
        mask = ((i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - w))[None].expand(B, -1, -1).contiguous()
        extra = None
        if holes:
            g = torch.Generator().manual_seed(seed)
            extra = torch.rand(B, N, N, generator=g) < 0.8
            extra[:, 5, :] = False                       # a dead query
            extra[:, 9, :] = False
            extra[:, 9, 9] = True                        # a query with a single visible key
            mask = mask & extra
        leaves = {n: xs[n].double().requires_grad_(True) for n in NAMES}
        exp = [leaves[n] if n == "Q" else leaves[n].expand(-1, Hq, -1, -1) for n in NAMES]
        Y, lse = tsg.reference(*exp, mask)
        Y.backward(dY.double())
        out = {"inputs": xs, "dY": dY, "window": w, "extra_mask": extra, "Y": Y.detach().float(),
               "lse": lse.detach().float()}
        for g, n in zip(["dQ", "dR", "dS", "dVr", "dVs"], NAMES):
            out[g] = leaves[n].grad.float()
        torch.save(out, HERE / f"shared_B{B}H{Hq}N{N}_s{seed}_w{w}{'_holes' if holes else ''}.pt")


def build_torch_reference(ref: Path):
    from torch.utils.cpp_extension import load
    build = REPO / "oracle" / "_ref" / "torch_reference_build"
    build.mkdir(parents=True, exist_ok=True)
    return load(name="att3_torch_reference", sources=[str(ref / "cpp" / "torch_reference.cpp")],
                build_directory=str(build), verbose=False)


HG_NAMES = ["Q", "R", "S", "Vq_1", "Vq_2", "Vr_1", "Vr_2", "Vs_1", "Vs_2"]


def hypergraph_cases(ref_ext, ttc):
    # unmasked: six outputs and nine gradients from cpp/torch_reference.cpp on BF16-rounded inputs
    for B, H, N, D, seed in [(1, 2, 16, 16, 0), (2, 2, 32, 32, 1), (1, 2, 48, 64, 2), (1, 1, 32, 128, 3)]:
        g = torch.Generator().manual_seed(seed)
        bf = {n: torch.randn(B, H, N, D, generator=g).to(torch.bfloat16) for n in HG_NAMES}
        gY = [torch.randn(B, H, N, D, generator=g).to(torch.bfloat16) for _ in range(6)]
        leaves = {n: v.double().requires_grad_(True) for n, v in bf.items()}
        outs = ref_ext.forward(*[leaves[n] for n in HG_NAMES], 0.0)
        sum((y * c.double()).sum() for y, c in zip(outs, gY)).backward()
        torch.save({"inputs": bf, "cotangents": gY, "outputs": [o.detach().float() for o in outs],
                    "grads": [leaves[n].grad.float() for n in HG_NAMES]},
                   HERE / f"hg_B{B}H{H}N{N}D{D}_s{seed}.pt")
    # masked gathers: tests/test_tc_paths.py::_ref_gather_masked with its own mask kinds
    for kind in ttc.MASK_KINDS:
        B, H, N, D = 2, 2, 32, 64
        g = torch.Generator().manual_seed(17)
        bf = {n: torch.randn(B, H, N, D, generator=g).to(torch.bfloat16) for n in HG_NAMES}
        gY = [torch.randn(B, H, N, D, generator=g).to(torch.bfloat16) for _ in range(3)]
        torch.manual_seed(5)
        mask = ttc._make_mask(kind, B, N, "cpu")
        leaves = {n: v.double().requires_grad_(True) for n, v in bf.items()}
        outs = ttc._ref_gather_masked(leaves["Q"], leaves["R"], leaves["S"], leaves["Vq_1"], leaves["Vr_1"],
                                      leaves["Vs_1"], mask)
        sum((y * c.double()).sum() for y, c in zip(outs, gY)).backward()
        grads = [leaves[n].grad.float() if leaves[n].grad is not None else torch.zeros(B, H, N, D) for n in HG_NAMES]
        torch.save({"inputs": bf, "cotangents": gY, "mask": mask, "outputs": [o.detach().float() for o in outs],
                    "grads": grads}, HERE / f"hg_masked_{kind}.pt")


def naive_c1(naive):
    """CPU naive reference at B2 N64 d_model64 H4 (d_head 16), fp32, no mask:
    x ~ N(0,1), Xavier-uniform projection weights from seed 0, dY ~ N(0,1)."""
    torch.manual_seed(0)
    mod = naive._HypergraphAttentionNaive(64, 4, head_subspaces=True)
    for name, prm in mod.named_parameters():
        if prm.dim() == 2:
            torch.nn.init.xavier_uniform_(prm)
    x = torch.randn(2, 64, 64, requires_grad=True)
    dY = torch.randn(2, 64, 64)
    y = mod(x, None)
    y.backward(dY)
    torch.save({"state_dict": {k: v.detach().clone() for k, v in mod.state_dict().items()}, "x": x.detach(), "dY": dY,
                "y": y.detach(), "dx": x.grad.clone(),
                "dW": {k: p.grad.clone() for k, p in mod.named_parameters() if p.grad is not None}},
               HERE / "naive_c1.pt")


def bounds(ref: Path):
    out_dir = REPO / "oracle" / "_ref"
    out_dir.mkdir(parents=True, exist_ok=True)
    exe = out_dir / "ref_bounds_dump"
    subprocess.run(["g++", "-O1", "-std=c++17", "-I/usr/local/cuda/include", f"-I{ref / 'cuda'}",
                    str(REPO / "oracle" / "ref_bounds_dump.cpp"), "-o", str(exe)], check=True)
    data = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    json.loads(data)
    (HERE / "bounds.json").write_text(data)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    a = ap.parse_args()
    ref = Path(a.reference)
    torch.set_num_threads(os.cpu_count())
    ref_ext = build_torch_reference(ref)
    mods = load_reference_modules(ref, ref_ext)
    single_gather_cases(mods["test_single_gather"])
    shared_cases(mods["test_single_gather"])
    hypergraph_cases(ref_ext, mods["test_tc_paths"])
    naive_c1(mods["naive"])
    bounds(ref)
    print("golden vectors written to", HERE)
