"""GPU parity tests of the windowed single gather (independent and shared KV heads).
Every call goes through the C ABI (``libatt3_b200.so``); the CPU oracle and the
golden vectors made from the reference's oracles are the checkers.  Gates are the
reference's: rel-L2 / max-norm (Y 0.03/0.05, dVr dVs 0.04/0.05, dQ dR dS 0.06/0.10),
|LSE| <= 0.02, identical dead-row sets, Y = 0 on dead rows
(tests/test_single_gather.py:26-30, 93-141)."""
import math

import pytest
import torch

from conftest import golden_files, load_golden
from oracle import triplet_oracle as O

pytestmark = pytest.mark.gpu

NAMES = ["Q", "R", "S", "Vr", "Vs"]
GRADS = ["dQ", "dR", "dS", "dVr", "dVs"]


@pytest.fixture(scope="module")
def ck():
    from att3ntion_b200 import _cuda_kernels
    return _cuda_kernels


def cuda(t):
    return None if t is None else t.cuda()


def run_lowlevel(ck, xs, dY, mask, window):
    q = [cuda(xs[n]) for n in NAMES]
    mk = cuda(mask)
    Y, m, l = ck.sg_forward_raw(*q, mk, window)
    grads = ck.sg_backward_raw(cuda(dY), *q, Y, m, l, mk, window)
    ck.device_status()
    return Y, m, l, dict(zip(GRADS, grads))


def check_all(Y, m, l, grads, ref):
    O.check_gate("Y", Y.float().cpu(), ref["Y"])
    O.check_lse(m, l, ref["lse"])
    dead = torch.isinf(ref["lse"])
    if dead.any():
        assert Y.cpu()[dead].abs().max().item() == 0.0, "dead query rows must produce Y = 0"
        assert (m.cpu()[dead] == -1e30).all() and (l.cpu()[dead] == 0).all()
    for g in GRADS:
        O.check_gate(g, grads[g].float().cpu(), ref[g])


def window_of(kind):
    return int(kind[6:]) if kind.startswith("window") else None


# --------------------------------------------------------------------------- golden vectors

WINDOWED_SG = [n for n in golden_files("sg_") if "_window" in n]


@pytest.mark.parametrize("name", WINDOWED_SG)
def test_windowed_golden_lowlevel(ck, name):
    g = load_golden(name)
    N = g["inputs"]["Q"].shape[2]
    if N % 16:
        pytest.skip("low-level entry points need N % 16 == 0; the bridge test covers this shape")
    w = window_of(g["kind"])
    # once with the window generated in-kernel, once with the dense mask the reference passes
    for mask in (None, g["mask"]):
        Y, m, l, grads = run_lowlevel(ck, g["inputs"], g["dY"], mask, w)
        check_all(Y, m, l, grads, g)


@pytest.mark.parametrize("name", WINDOWED_SG)
def test_windowed_golden_bridge(name):
    from att3ntion_b200 import single_gather_attention
    g = load_golden(name)
    w = window_of(g["kind"])
    leaves = {n: g["inputs"][n].cuda().requires_grad_(True) for n in NAMES}
    Y = single_gather_attention(*[leaves[n] for n in NAMES], None, w)
    Y.backward(g["dY"].cuda())
    O.check_gate("Y", Y.detach().float().cpu(), g["Y"])
    for gname, n in zip(GRADS, NAMES):
        O.check_gate(gname, leaves[n].grad.float().cpu(), g[gname])


@pytest.mark.parametrize("name", golden_files("shared_"))
def test_shared_golden_bridge(name):
    from att3ntion_b200 import single_gather_shared_attention
    g = load_golden(name)
    leaves = {n: g["inputs"][n].cuda().requires_grad_(True) for n in NAMES}
    Y = single_gather_shared_attention(*[leaves[n] for n in NAMES], cuda(g["extra_mask"]), window=g["window"])
    Y.backward(g["dY"].cuda())
    O.check_gate("Y", Y.detach().float().cpu(), g["Y"])
    dead = torch.isinf(g["lse"])
    if dead.any():
        assert Y.detach().cpu()[dead].abs().max().item() == 0.0
    for gname, n in zip(GRADS, NAMES):
        grad = leaves[n].grad
        assert grad.shape == g[gname].shape
        O.check_gate(gname, grad.float().cpu(), g[gname])


# --------------------------------------------------------------------------- seeded cases vs the oracle

def draw(B, Hq, Hkv, N, D, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    xs = {"Q": (torch.randn(B, Hq, N, D, generator=g) * scale).to(torch.bfloat16)}
    for n in NAMES[1:]:
        xs[n] = (torch.randn(B, Hkv, N, D, generator=g) * scale).to(torch.bfloat16)
    dY = (torch.randn(B, Hq, N, D, generator=g) * scale).to(torch.bfloat16)
    return xs, dY


@pytest.mark.parametrize("window", [16, 32, 64, 128])
@pytest.mark.parametrize("N", [16, 64, 144, 272])
@pytest.mark.parametrize("Hq,Hkv,D", [(4, 1, 128), (2, 2, 64), (4, 2, 128)])
def test_windows_and_lengths(ck, window, N, Hq, Hkv, D):
    xs, dY = draw(2, Hq, Hkv, N, D, seed=N + window)
    ref = O.single_gather_banded(*[xs[n] for n in NAMES], window=window, dY=dY, chunk=48)
    Y, m, l, grads = run_lowlevel(ck, xs, dY, None, window)
    check_all(Y, m, l, grads, ref)


@pytest.mark.parametrize("scale", [0.5, 1.0])
def test_extra_mask_dead_and_singleton_rows(ck, scale):
    B, Hq, N, D, w = 2, 4, 96, 128, 32
    xs, dY = draw(B, Hq, 1, N, D, seed=5, scale=scale)
    g = torch.Generator().manual_seed(1)
    extra = torch.rand(B, N, N, generator=g) < 0.7
    extra[:, 7, :] = False                                   # dead query
    extra[:, 40, :] = False
    extra[:, 40, 40] = True                                  # singleton query
    ref = O.single_gather_banded(*[xs[n] for n in NAMES], window=w, dY=dY, mask=extra, chunk=32)
    Y, m, l, grads = run_lowlevel(ck, xs, dY, extra, w)
    check_all(Y, m, l, grads, ref)
    assert grads["dQ"][:, :, 7].abs().max().item() == 0.0
    # one visible key: exactly zero score gradients for that query (tests/test_shared_auto.py:17-32)
    assert grads["dQ"][:, :, 40].abs().max().item() == 0.0


@pytest.mark.parametrize("Hq,Hkv", [(1, 1), (8, 1)])
def test_long_sequence_one_and_many_heads_per_key_head(ck, Hq, Hkv):
    """Many query boundaries in one CTA, with one head per query (the H warps run several queries
    ahead of the ring updates) and with eight."""
    xs, dY = draw(1, Hq, Hkv, 1536 if Hq == 1 else 640, 128, seed=21)
    ref = O.single_gather_banded(*[xs[n] for n in NAMES], window=128, dY=dY, chunk=64)
    Y, m, l, grads = run_lowlevel(ck, xs, dY, None, 128)
    check_all(Y, m, l, grads, ref)


@pytest.mark.parametrize("Hq", [1, 4])
def test_runs_of_dead_queries_between_live_ones(ck, Hq):
    """Queries without any visible key in runs of one to five, also around multiples of 128: the
    boundary duties (ring rows, accumulator flush) of queries that launch no MMA."""
    B, N, D, w = 1, 400, 128, 64
    xs, dY = draw(B, Hq, 1, N, D, seed=31)
    mask = torch.ones(B, N, N, dtype=torch.bool)
    for start, run in ((5, 1), (60, 3), (126, 5), (255, 2), (300, 4), (396, 4)):
        mask[:, start:start + run, :] = False
    ref = O.single_gather_banded(*[xs[n] for n in NAMES], window=w, dY=dY, mask=mask, chunk=40)
    Y, m, l, grads = run_lowlevel(ck, xs, dY, mask, w)
    check_all(Y, m, l, grads, ref)
    dead = ~mask.any(-1)[0]
    assert Y[:, :, dead].abs().max().item() == 0.0
    assert grads["dQ"][:, :, dead].abs().max().item() == 0.0


def test_all_masked_gives_zeros(ck):
    xs, dY = draw(1, 2, 1, 32, 128, seed=2)
    mask = torch.zeros(1, 32, 32, dtype=torch.bool)
    Y, m, l, grads = run_lowlevel(ck, xs, dY, mask, 16)
    assert Y.abs().max().item() == 0.0 and (l == 0).all() and (m == -1e30).all()
    for g in GRADS:
        assert grads[g].abs().max().item() == 0.0


def test_single_head_cotangent_isolation(ck):
    """dY on one head only: the other heads' dQ must be exactly zero."""
    xs, dY = draw(1, 4, 1, 64, 128, seed=9)
    dY[:, [0, 1, 3]] = 0
    Y, m, l, grads = run_lowlevel(ck, xs, dY, None, 32)
    assert grads["dQ"][:, [0, 1, 3]].abs().max().item() == 0.0
    assert grads["dQ"][:, 2].abs().max().item() > 0.0


def test_repeated_calls_are_bit_identical(ck):
    xs, dY = draw(2, 8, 1, 400, 128, seed=3)
    a = run_lowlevel(ck, xs, dY, None, 128)
    b = run_lowlevel(ck, xs, dY, None, 128)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    for g in GRADS:
        assert torch.equal(a[3][g], b[3][g]), g


def test_row_shard_with_halo_equals_full_run(ck):
    """Queries [q_begin, N) computed from a slice that starts (w-1) keys earlier give
    the same rows as the full sequence: the property row sharding across GPUs rests on."""
    w, N, cut = 64, 384, 208
    xs, dY = draw(1, 4, 1, N, 128, seed=4)
    q = [xs[n].cuda() for n in NAMES]
    Y, m, l = ck.sg_forward_raw(*q, None, w)
    full = ck.sg_backward_raw(dY.cuda(), *q, Y, m, l, None, w)
    # The slice starts at a multiple of 128, so every key keeps its ring slot and the
    # contractions sum in the same order: the shard's rows are then bit-identical.
    lo = 128                                               # 80 >= w - 1 halo rows in front of `cut`
    qs = [t[:, :, lo:].contiguous() for t in q]
    Ys, ms, ls = ck.sg_forward_raw(*qs, None, w, q_begin=cut - lo)
    assert torch.equal(Ys[:, :, cut - lo:], Y[:, :, cut:])
    assert torch.equal(ms[:, :, cut - lo:], m[:, :, cut:]) and torch.equal(ls[:, :, cut - lo:], l[:, :, cut:])
    part = ck.sg_backward_raw(dY.cuda()[:, :, lo:].contiguous(), *qs, Ys, ms, ls, None, w, q_begin=cut - lo)
    assert torch.equal(part[0][:, :, cut - lo:], full[0][:, :, cut:])            # dQ rows
    # KV gradients of the upper shard + those of the lower shard = the full gradients
    qlow = [t[:, :, :cut].contiguous() for t in q]
    Yl, ml, ll = ck.sg_forward_raw(*qlow, None, w)
    low = ck.sg_backward_raw(dY.cuda()[:, :, :cut].contiguous(), *qlow, Yl, ml, ll, None, w)
    for k in range(1, 5):
        total = torch.zeros_like(full[k], dtype=torch.float32)
        total[:, :, :cut] += low[k].float()
        total[:, :, lo:] += part[k].float()
        rel, mx = O.errors(total, full[k].float())
        assert rel < 0.01 and mx < 0.02, (k, rel, mx)
    ck.device_status()


def test_non_default_stream_and_graph_replay(ck):
    xs, dY = draw(1, 4, 1, 128, 128, seed=6)
    q = [xs[n].cuda() for n in NAMES]
    dYc = dY.cuda()
    Y0, m0, l0 = ck.sg_forward_raw(*q, None, 64)
    g0 = ck.sg_backward_raw(dYc, *q, Y0, m0, l0, None, 64)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        Y1, m1, l1 = ck.sg_forward_raw(*q, None, 64)
        g1 = ck.sg_backward_raw(dYc, *q, Y1, m1, l1, None, 64)
    s.synchronize()
    assert torch.equal(Y0, Y1) and all(torch.equal(a, b) for a, b in zip(g0, g1))
    # CUDA-graph capture and replay (tests/test_shared_auto.py:61-75): no host sync in the path
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        ck.sg_backward_raw(dYc, *q, Y0, m0, l0, None, 64)       # warm the workspace outside capture
        s.synchronize()
        with torch.cuda.graph(graph, stream=s):
            Y2, m2, l2 = ck.sg_forward_raw(*q, None, 64)
            g2 = ck.sg_backward_raw(dYc, *q, Y2, m2, l2, None, 64)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(Y0, Y2) and all(torch.equal(a, b) for a, b in zip(g0, g2))


def test_lowlevel_rejections(ck):
    xs, dY = draw(1, 8, 1, 32, 128, seed=1)
    q = [xs[n].cuda() for n in NAMES]
    mask = O.window_mask(32, 32)[None].cuda().contiguous()
    with pytest.raises(RuntimeError, match="mask must be"):
        ck.single_gather_shared_forward(*q, None, 32, 1)          # the low-level binding needs its mask
    with pytest.raises(RuntimeError, match="window must be"):
        ck.single_gather_shared_forward(*q, mask, 48, 1)
    with pytest.raises(RuntimeError, match="head group"):
        ck.single_gather_shared_forward(*q, mask, 32, 3)
    with pytest.raises(RuntimeError, match="KV tensors must be"):
        ck.single_gather_shared_forward(q[0], q[0], q[2], q[3], q[4], mask, 32, 1)
    with pytest.raises(RuntimeError, match="empty batch/head"):
        ck.single_gather_shared_forward(q[0][:0], *q[1:], mask, 32, 1)
    Y, m, l = ck.single_gather_shared_forward(*q, mask, 32, 1)
    with pytest.raises(RuntimeError, match="Q's device"):
        ck.single_gather_shared_backward(dY.cuda(), *q, Y, m.cpu(), l, mask, 32, 1)
    before = ck.tc_launches()["sg_forward"]
    ck.single_gather_shared_forward(*q, mask, 32, 2)
    assert ck.tc_launches()["sg_forward"] == before + 1
    assert "win=32" in ck.sg_dispatch()["shared_forward"]


def test_head_split_partials_sum_to_the_full_key_gradients(ck):
    """Query heads split in two (as two GPUs of one batch shard would hold them): Y and dQ of each half are
    bit-identical to the full run's slices, and the FP32 key-gradient partials of the halves add up to the
    full run's key gradients (summation order differs, so to FP32 rounding before the final BF16 rounding)."""
    B, Hq, N, D, w = 2, 8, 400, 128, 128
    g = torch.Generator(device="cpu").manual_seed(17)
    Q = (torch.randn(B, Hq, N, D, generator=g) / math.sqrt(D)).to(torch.bfloat16).cuda()
    kv = [(torch.randn(B, 1, N, D, generator=g) / math.sqrt(D)).to(torch.bfloat16).cuda() for _ in range(4)]
    dY = torch.randn(B, Hq, N, D, generator=g).to(torch.bfloat16).cuda()
    Y, m, l = ck.sg_forward_raw(Q, *kv, None, w)
    full = ck.sg_backward_raw(dY, Q, *kv, Y, m, l, None, w)
    parts = []
    for heads in (slice(0, 4), slice(4, 8)):
        Qh, dYh = Q[:, heads].contiguous(), dY[:, heads].contiguous()
        Yh, mh, lh = ck.sg_forward_raw(Qh, *kv, None, w)
        assert torch.equal(Yh, Y[:, heads]) and torch.equal(mh, m[:, heads]) and torch.equal(lh, l[:, heads])
        gh = ck.sg_backward_raw(dYh, Qh, *kv, Yh, mh, lh, None, w, kv_f32=True)
        assert gh[1].dtype == torch.float32
        assert torch.equal(gh[0], full[0][:, heads])
        parts.append(gh)
    ck.device_status()
    for k in range(1, 5):
        total = (parts[0][k] + parts[1][k])
        rel, mx = O.errors(total, full[k].float())
        assert rel < 4e-3 and mx < 8e-3, (k, rel, mx)       # BF16 rounding of the full run's output only


def test_full_size_properties_c4_shape(ck):
    """Shared-KV B4 Hq8 N8192 D128 w128: too large for the dense oracle, so check
    (i) a 192-query slice of one batch against the banded FP64 oracle (Y, LSE, dQ
    and the 65 complete rows of the four key gradients), (ii) that
    interior rows are invariant to shifting the sequence by one window, and
    (iii) repeat-call equality of the KV gradients."""
    B, Hq, N, D, w = 4, 8, 8192, 128, 128
    g = torch.Generator(device="cpu").manual_seed(3)
    Q = (torch.randn(B, Hq, N, D, generator=g) / math.sqrt(D)).to(torch.bfloat16)
    kv = [(torch.randn(B, 1, N, D, generator=g) / math.sqrt(D)).to(torch.bfloat16) for _ in range(4)]
    dY = torch.randn(B, Hq, N, D, generator=g).to(torch.bfloat16)
    q = [Q.cuda()] + [t.cuda() for t in kv]
    Y, m, l = ck.sg_forward_raw(*q, None, w)
    grads = ck.sg_backward_raw(dY.cuda(), *q, Y, m, l, None, w)
    ck.device_status()
    lo, hi, b = 4000, 4192, 2
    sl = slice(lo - 127, hi)
    ref = O.single_gather_banded(Q[b:b + 1, :, sl], *[t[b:b + 1, :, sl] for t in kv], window=w,
                                 dY=dY[b:b + 1, :, sl], q_begin=127, chunk=32)
    O.check_gate("Y", Y[b:b + 1, :, lo:hi].float().cpu(), ref["Y"][:, :, 127:])
    O.check_lse(m[b:b + 1, :, lo:hi], l[b:b + 1, :, lo:hi], ref["lse"][:, :, 127:])
    O.check_gate("dQ", grads[0][b:b + 1, :, lo:hi].float().cpu(), ref["dQ"][:, :, 127:])
    # key k collects from queries k .. k+127: the slice holds all of them for keys lo .. hi-128, so the head-summed
    # key gradients of those rows are complete in the oracle (partial planes + reduction at full size)
    nk = hi - lo - 127
    for gi, gname in enumerate(["dR", "dS", "dVr", "dVs"], start=1):
        O.check_gate(gname, grads[gi][b:b + 1, :, lo:lo + nk].float().cpu(), ref[gname][:, :, 127:127 + nk])
    # shift invariance: drop the first 128 positions, rows >= 255 of the original are unchanged
    qs = [t[:, :, 128:].contiguous() for t in q]
    Ys, ms, ls = ck.sg_forward_raw(*qs, None, w)
    assert torch.equal(Ys[:, :, 127:], Y[:, :, 255:])
    again = ck.sg_backward_raw(dY.cuda(), *q, Y, m, l, None, w)
    assert all(torch.equal(a, b2) for a, b2 in zip(grads, again))
    for t in grads:
        assert torch.isfinite(t).all()
