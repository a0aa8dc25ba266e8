"""Semantic gates of the reference's test-suite that do not depend on its schedules, restated against
this implementation: boundary lengths through the bridge (tests/test_single_gather.py:406-427),
bit-equality of a window-only call and the same call with the window given as a mask (381-400),
device switching (tests/test_shared_auto.py:46-59), CUDA-graph replay of the shared-KV binding-level
functions (61-75), the stress distributions (tests/test_single_gather.py:487-520) and the two
self-tests of the library (operand descriptors, bounded waits)."""
import math

import pytest
import torch

from oracle import triplet_oracle as O

pytestmark = pytest.mark.gpu

NAMES = ["Q", "R", "S", "Vr", "Vs"]
GRADS = ["dQ", "dR", "dS", "dVr", "dVs"]


@pytest.fixture(scope="module")
def ck():
    from att3ntion_b200 import _cuda_kernels
    return _cuda_kernels


def draw(B, H, N, D, seed, scale=1.0, hkv=None):
    g = torch.Generator(device="cpu").manual_seed(seed)
    xs = {"Q": (torch.randn(B, H, N, D, generator=g) * scale).to(torch.bfloat16)}
    for n in NAMES[1:]:
        xs[n] = (torch.randn(B, hkv or H, N, D, generator=g) * scale).to(torch.bfloat16)
    dY = torch.randn(B, H, N, D, generator=g).to(torch.bfloat16)
    return xs, dY


def make_mask(kind, B, N, seed=0):
    """Mask kinds of tests/test_single_gather.py:34-49."""
    if kind == "none":
        return None
    i = torch.arange(N)
    if kind == "causal":
        m = i[None, :] <= i[:, None]
    elif kind == "window16":
        m = (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - 16)
    elif kind == "random_dead":
        g = torch.Generator(device="cpu").manual_seed(seed)
        m = torch.rand(B, N, N, generator=g) < 0.6
        m[:, N // 2, :] = False
        return m
    return m[None].expand(B, -1, -1).contiguous()


def bridge(xs, dY, mask, window):
    from att3ntion_b200 import single_gather_attention
    leaves = {n: xs[n].cuda().requires_grad_(True) for n in NAMES}
    Y = single_gather_attention(*[leaves[n] for n in NAMES], None if mask is None else mask.cuda(), window=window)
    Y.backward(dY.cuda())
    return Y.detach(), {g: leaves[n].grad for g, n in zip(GRADS, NAMES)}


def check(Y, grads, ref):
    O.check_gate("Y", Y.float().cpu(), ref["Y"])
    dead = torch.isinf(ref["lse"])
    if dead.any():
        assert Y.cpu()[dead].abs().max().item() == 0.0
    for g in GRADS:
        O.check_gate(g, grads[g].float().cpu(), ref[g])


# --------------------------------------------------------------------------- boundary lengths through the bridge

BOUNDARY_N = [15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257]
_KINDS = ["causal", "window16", "none", "random_dead"]
_SHAPES = [(1, 2), (2, 1), (1, 3)]
BOUNDARY = [(N, 64 if i % 2 == 0 else 128, _KINDS[i % 4], *_SHAPES[i % 3]) for i, N in enumerate(BOUNDARY_N)]


@pytest.mark.parametrize("N,D,kind,B,H", BOUNDARY)
def test_boundary_lengths(N, D, kind, B, H):
    xs, dY = draw(B, H, N, D, 13)
    mask = make_mask(kind, B, N, 13)
    ref = O.single_gather_dense(*[xs[n] for n in NAMES], mask=mask, dY=dY)
    window = {"causal": N, "window16": 16}.get(kind, 0)
    for win in ({0, window} if window else {0}):
        Y, grads = bridge(xs, dY, mask, win)
        check(Y, grads, ref)


@pytest.mark.parametrize("N", [33, 65, 100])
def test_window_only_call_equals_the_call_with_the_window_as_a_mask(N):
    """Both calls run the same kernel on the same visibility, so their results are bit-identical."""
    B, H, D, w = 1, 2, 64, 16
    xs, dY = draw(B, H, N, D, 9)
    mask = O.window_mask(N, w)[None].expand(B, -1, -1).contiguous()
    ref = O.single_gather_dense(*[xs[n] for n in NAMES], mask=mask, dY=dY)
    Ya, ga = bridge(xs, dY, None, w)
    Yb, gb = bridge(xs, dY, mask, w)
    assert torch.equal(Ya, Yb)
    for g in GRADS:
        assert torch.equal(ga[g], gb[g]), g
    check(Ya, ga, ref)


# --------------------------------------------------------------------------- devices and graphs

@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="requires two CUDA devices")
@pytest.mark.parametrize("window", [16, 32, 64, 128])
def test_one_library_can_switch_devices(ck, window):
    xs, dY = draw(1, 16, 128, 128, seed=193, hkv=1)
    reference = None
    for device in (0, 1, 0):
        with torch.cuda.device(device):
            q = [xs[n].to(f"cuda:{device}") for n in NAMES]
            Y, m, l = ck.sg_forward_raw(*q, None, window)
            grads = ck.sg_backward_raw(dY.to(f"cuda:{device}"), *q, Y, m, l, None, window)
            ck.device_status(f"cuda:{device}")
            got = [t.cpu() for t in (Y, m, l, *grads)]
        if reference is None:
            reference = got
        else:
            assert all(torch.equal(a, b) for a, b in zip(reference, got))


def test_shared_binding_functions_replay_in_a_cuda_graph(ck):
    xs, dY = draw(1, 8, 256, 128, seed=197, hkv=1)
    q = [xs[n].cuda() for n in NAMES]
    dYc = dY.cuda()
    mask = O.window_mask(256, 32)[None].contiguous().cuda()

    def step():
        out = ck.single_gather_shared_forward(*q, mask, 32, 0)
        return out, ck.single_gather_shared_backward(dYc, *q, *out, mask, 32, 0)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            eager = step()
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            out, grads = step()
    graph.replay()
    torch.cuda.synchronize()
    saved = [t.clone() for t in (*out, *grads)]
    graph.replay()
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(saved, (*out, *grads)))
    assert all(torch.equal(a, b) for a, b in zip(saved, (*eager[0], *eager[1])))
    ck.device_status()


# --------------------------------------------------------------------------- stress distributions

DISTS = ["scale0.25", "scale4", "dy1e-3", "dy1e3", "concentrated", "uniform", "cancel"]
# Cases outside the reference's own gates with these kernels (BF16 operands, FP32 accumulation), recorded so
# that a change in the set shows up; the reference records its own failing stress cases the same way
# (docs/KERNEL_HISTORY.md:21: scaled inputs and concentrated softmaxes, "BF16 rounding of products ... before
# tensor-core GEMMs").  The pattern here: with scores of magnitude ~50 and more, the BF16 rounding of the
# Hadamard operand moves a score by a few tenths; the pass that produces dR, dVr rounds Q o S where the
# forward (whose statistics it uses) rounded Q o R, so its probabilities are normalised with statistics that
# belong to slightly different scores.  dS, dVs share the forward's rounding and stay inside the gates in the
# "concentrated" cases.  Key: (D, distribution, seed) -> gradients outside the gates.
KNOWN_STRESS_FAILURES = {
    (64, "scale4", 0): ["Y", "dQ", "dR", "dS", "dVr"],
    (64, "scale4", 1): ["Y", "dQ", "dR", "dS", "dVr", "dVs"],
    (64, "concentrated", 0): ["dR", "dVr"],
    (64, "concentrated", 1): ["dR", "dVr"],
    (128, "scale4", 0): ["dQ", "dR", "dS", "dVr"],
    (128, "scale4", 1): ["Y", "dQ", "dR", "dS", "dVr", "dVs"],
    (128, "concentrated", 0): ["dQ", "dR", "dS", "dVr"],      # dQ, dS: one head just over its per-head gate
    (128, "concentrated", 1): ["dR", "dVr"],
}


def draw_dist(B, H, N, D, seed, dist):
    g = torch.Generator(device="cpu").manual_seed(seed)
    s_qrs, s_v, s_dy = {"scale0.25": (0.25, 0.25, 1.0), "scale4": (4.0, 4.0, 1.0), "dy1e-3": (1.0, 1.0, 1e-3),
                        "dy1e3": (1.0, 1.0, 1e3), "concentrated": (3.0, 1.0, 1.0), "uniform": (0.05, 1.0, 1.0),
                        "cancel": (1.0, 1.0, 1.0)}[dist]
    xs = {}
    for n in NAMES:
        sc = s_qrs if n in ("Q", "R", "S") else s_v
        xs[n] = (torch.randn(B, H, N, D, generator=g) * sc).to(torch.bfloat16)
    if dist == "cancel":        # values with a large common offset: Y is a small difference of big numbers
        xs["Vr"] = (xs["Vr"].float() + 8.0).to(torch.bfloat16)
        xs["Vs"] = (xs["Vs"].float() - 8.0).to(torch.bfloat16)
    dY = (torch.randn(B, H, N, D, generator=g) * s_dy).to(torch.bfloat16)
    return xs, dY


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dist", DISTS)
@pytest.mark.parametrize("seed", [0, 1])
def test_stress_distributions(D, dist, seed):
    B, H, N = 1, 2, 65
    xs, dY = draw_dist(B, H, N, D, seed, dist)
    mask = make_mask("causal", B, N)
    ref = O.single_gather_dense(*[xs[n] for n in NAMES], mask=mask, dY=dY)
    Y, grads = bridge(xs, dY, mask, N)
    failed = []
    for name, t in [("Y", Y)] + [(g, grads[g]) for g in GRADS]:
        try:
            O.check_gate(name, t.float().cpu(), ref[name])
        except AssertionError:
            failed.append(name)
    expected = KNOWN_STRESS_FAILURES.get((D, dist, seed), [])
    if sorted(failed) != sorted(expected):
        pytest.fail(f"stress case (D={D}, {dist}, seed {seed}): outside the gates {sorted(failed)}, recorded {sorted(expected)}")
    if failed:
        pytest.xfail(f"recorded stress failure: {failed}")


# --------------------------------------------------------------------------- library self-tests

@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4, 8, 11, 12])
def test_operand_descriptor_encodings(mode):
    """Each operand arrangement the kernels use (K-major / MN-major shared memory, A in tensor memory), with the
    encodings fixed inside the library, against a plain matrix product."""
    from att3ntion_b200 import _cabi
    torch.manual_seed(0)
    A = torch.randn(128, 128, device="cuda").bfloat16()
    Bm = torch.randn(128, 128, device="cuda").bfloat16()
    Af, Bf = A.float(), Bm.float()
    ref = {0: Af @ Bf.T, 1: Af @ Bf, 2: Af.T @ Bf, 3: Af @ Bf, 4: Af @ Bf.T}[mode & 7]
    Dm = torch.full((128, 128), float("nan"), device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    _cabi.check(_cabi.lib.att3_umma_selftest(A.data_ptr(), Bm.data_ptr(), Dm.data_ptr(), mode, st.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert st[0].item() == 0, "the bounded wait for the product ran out"
    cols = 64 if mode & 8 else 128
    assert (Dm[:, :cols] - ref[:, :cols]).abs().max().item() < 1e-3
    if mode & 8:
        assert torch.isnan(Dm[:, 64:]).all()


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(ck):
    """One thread waits, for a bounded number of polls, on a barrier nobody arrives on; the kernel returns
    normally, the status word says so, and the next kernels run as if nothing had happened."""
    from att3ntion_b200 import _cabi
    lib = _cabi.lib
    ck.device_status()                                                   # start from a clean word
    _cabi.check(lib.att3_wait_selftest(2000, torch.cuda.current_stream().cuda_stream))
    rc = lib.att3_device_status(torch.cuda.current_stream().cuda_stream)
    assert rc == _cabi.ERR_TIMEOUT and "bounded device-side wait" in _cabi.last_error()
    assert lib.att3_device_status(torch.cuda.current_stream().cuda_stream) == _cabi.OK      # read clears it
    xs, dY = draw(1, 2, 64, 128, seed=1, hkv=1)
    q = [xs[n].cuda() for n in NAMES]
    Y, m, l = ck.sg_forward_raw(*q, None, 32)
    ck.sg_backward_raw(dY.cuda(), *q, Y, m, l, None, 32)
    ck.device_status()
    assert torch.isfinite(Y.float()).all()
    assert lib.att3_wait_selftest(0, None) == _cabi.ERR_INVALID


# --------------------------------------------------------------------------- extended calls: packed masks, window pairs

def test_packed_mask_words_equal_the_byte_mask(ck):
    """The same mask as bytes and as packed words gives bit-identical results on both windowed schedules
    (ring: w = 128; packed tiles: w = 32), and the packer's words / support counts match a torch restatement."""
    B, Hq, N, D = 2, 4, 208, 128
    xs, dY = draw(B, Hq, N, D, seed=41, hkv=1)
    g = torch.Generator().manual_seed(2)
    mask = torch.rand(B, N, N, generator=g) < 0.7
    mask[:, 9, :] = False
    mask[:, 77, :] = False
    mask[:, 77, 77] = True
    q = [xs[n].cuda() for n in NAMES]
    mk = mask.cuda().contiguous()
    for w in (128, 32):
        words, support = ck.pack_mask(mk, window=w, with_support=True)
        i = torch.arange(N)
        vis = mask & (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - w)
        assert torch.equal(support.cpu(), vis.sum(-1).clamp(max=2).to(torch.uint8))
        bits = torch.nn.functional.pad(vis, (0, (-N) % 32)).reshape(B, N, -1, 32).long()
        want = (bits << torch.arange(32)).sum(-1)
        assert torch.equal(words.cpu().long() & 0xFFFFFFFF, want)
        plain = ck.pack_mask(mk)                                          # the mask alone; the kernels apply the window
        Y0, m0, l0 = ck.sg_forward_raw(*q, mk, w)
        g0 = ck.sg_backward_raw(dY.cuda(), *q, Y0, m0, l0, mk, w)
        Y1, m1, l1 = ck.sg_forward_raw(*q, None, w, mask_words=plain)
        g1 = ck.sg_backward_raw(dY.cuda(), *q, Y1, m1, l1, None, w, mask_words=plain)
        ck.device_status()
        assert torch.equal(Y0, Y1) and torch.equal(m0, m1) and torch.equal(l0, l1)
        assert all(torch.equal(a, b) for a, b in zip(g0, g1))
        ref = O.single_gather_banded(*[xs[n] for n in NAMES], window=w, dY=dY, mask=mask, chunk=40)
        O.check_gate("Y", Y1.float().cpu(), ref["Y"])
        O.check_lse(m1, l1, ref["lse"])
        for name, t in zip(GRADS, g1):
            O.check_gate(name, t.float().cpu(), ref[name])
    with pytest.raises(RuntimeError, match="either as bytes or as packed words"):
        ck.sg_forward_raw(*q, mk, 32, mask_words=ck.pack_mask(mk))
    with pytest.raises(RuntimeError, match="windowed path"):
        ck.sg_forward_raw(*[xs[n][:, :1].expand(-1, 4, -1, -1).contiguous().cuda() if n != "Q" else q[0] for n in NAMES],
                          None, 0, mask_words=ck.pack_mask(mk))


@pytest.mark.parametrize("wr,ws", [(128, 32), (16, 96), (48, 48), (1, 128)])
def test_one_window_per_key_axis(wr, ws):
    """window = (w_r, w_s): query i sees the pairs (j, k) with j in (i - w_r, i] and k in (i - w_s, i]."""
    from att3ntion_b200 import single_gather_attention
    B, H, N, D = 1, 2, 200, 128
    xs, dY = draw(B, H, N, D, seed=wr + ws)
    mr = O.window_mask(N, wr)[None].expand(B, -1, -1)
    ms = O.window_mask(N, ws)[None].expand(B, -1, -1)
    ref = O.single_gather_dense(*[xs[n] for n in NAMES], mask=mr, dY=dY, mask_s=ms)
    leaves = {n: xs[n].cuda().requires_grad_(True) for n in NAMES}
    Y = single_gather_attention(*[leaves[n] for n in NAMES], None, window=(wr, ws))
    Y.backward(dY.cuda())
    check(Y.detach(), {g: leaves[n].grad for g, n in zip(GRADS, NAMES)}, ref)
    if wr == ws:        # a pair of equal windows is the plain windowed call
        Yb, gb = bridge(xs, dY, None, wr)
        assert torch.equal(Y.detach(), Yb)


@pytest.mark.parametrize("Hq,Hkv,D,w", [(8, 1, 128, 128), (8, 1, 128, 32), (4, 4, 64, 64), (2, 2, 128, 48)])
def test_heads_last_layout_and_activated_output(ck, Hq, Hkv, D, w):
    """Operands laid out [B,N,H,D] give, element for element, what the [B,H,N,D] call gives (both windowed schedules
    and both head sizes), and the activated output equals QuickGELU of the plain one."""
    B, N = 2, 272
    xs, dY = draw(B, Hq, N, D, seed=Hq + w, hkv=Hkv)
    q = [xs[n].cuda() for n in NAMES]
    Y0, m0, l0 = ck.sg_forward_raw(*q, None, w)
    g0 = ck.sg_backward_raw(dY.cuda(), *q, Y0, m0, l0, None, w)
    t = lambda x: x.permute(0, 2, 1, 3).contiguous()
    qt = [t(x) for x in q]
    Y1, m1, l1, Ya = ck.sg_forward_raw(*qt, None, w, bnhd=True, act=True)
    g1 = ck.sg_backward_raw(t(dY.cuda()), *qt, Y1, m1, l1, None, w, bnhd=True)
    ck.device_status()
    assert torch.equal(t(Y0), Y1) and torch.equal(m0, m1) and torch.equal(l0, l1)
    for a, b in zip(g0, g1):
        assert torch.equal(t(a), b)
    yf = Y1.float()
    assert torch.allclose(Ya.float(), yf * torch.sigmoid(1.702 * yf), rtol=2e-2, atol=1e-3)


def test_module_window_path_reads_projections_in_place():
    """HypergraphAttention(gather_mode=1, window): the path without permute-and-copy and with the fused activation
    agrees with the path through single_gather_attention + QuickGELU (same kernels, other memory layout)."""
    from att3ntion_b200 import HypergraphAttention
    from att3ntion_b200 import _autograd
    torch.manual_seed(0)
    mod = HypergraphAttention(256, 2, gather_mode=1, window=64).cuda()
    x = torch.randn(2, 96, 256, device="cuda", requires_grad=True)
    y = mod(x)
    y.sum().backward()
    gx, gw = x.grad.clone(), mod.Wq.weight.grad.clone()
    x.grad = None
    mod.zero_grad()
    tile = _autograd.TILE
    _autograd.TILE = 10 ** 9                       # n % TILE != 0: forces the permute-and-copy path
    try:
        y2 = mod(x)
        y2.sum().backward()
    finally:
        _autograd.TILE = tile
    assert torch.allclose(y, y2, rtol=2e-2, atol=2e-2)
    assert torch.allclose(gx, x.grad, rtol=5e-2, atol=5e-2) and torch.allclose(gw, mod.Wq.weight.grad, rtol=5e-2, atol=5e-1)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dist", ["scale4", "concentrated"])
@pytest.mark.parametrize("seed", [0, 1])
def test_compensated_products_pass_the_stress_gates(D, dist, seed):
    """precise=True: the score product on the exact split of Q o R.  The two stress distributions whose scores are
    large enough for the BF16 rounding of that operand to matter (and which fail without it, above) pass the
    reference's gates."""
    from att3ntion_b200 import single_gather_attention
    B, H, N = 1, 2, 65
    xs, dY = draw_dist(B, H, N, D, seed, dist)
    mask = make_mask("causal", B, N)
    ref = O.single_gather_dense(*[xs[n] for n in NAMES], mask=mask, dY=dY)
    leaves = {n: xs[n].cuda().requires_grad_(True) for n in NAMES}
    Y = single_gather_attention(*[leaves[n] for n in NAMES], mask.cuda(), window=N, precise=True)
    Y.backward(dY.cuda())
    check(Y.detach(), {g: leaves[n].grad for g, n in zip(GRADS, NAMES)}, ref)


def test_compensated_products_on_the_shared_kv_operator():
    from att3ntion_b200 import single_gather_shared_attention
    xs, dY = draw(2, 8, 400, 128, seed=77, hkv=1, scale=1.5)
    ref = O.single_gather_banded(*[xs[n] for n in NAMES], window=128, dY=dY, chunk=40)
    leaves = {n: xs[n].cuda().requires_grad_(True) for n in NAMES}
    Y = single_gather_shared_attention(*[leaves[n] for n in NAMES], None, window=128, precise=True)
    Y.backward(dY.cuda())
    check(Y.detach(), {g: leaves[n].grad for g, n in zip(GRADS, NAMES)}, ref)
