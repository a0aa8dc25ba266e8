"""Host shim over the C ABI with the surface of the reference's pybind module
``att3ntion._cuda_kernels`` (cpp/cuda_bindings.cpp:30-233): same function names,
argument order, return tuples and error behaviour (RuntimeError for rejected
tensors, ValueError for an unknown config key).  The shim validates tensors,
allocates the outputs with torch on the inputs' device, and passes raw device
pointers plus torch's current stream to ``libatt3_b200.so``.  There is no other
compute path: without the library the import of ``_cabi`` fails.
"""
from __future__ import annotations

import ctypes as C
import threading

import torch

from . import _cabi
from ._cabi import lib

_BF16 = torch.bfloat16
_state = threading.local()
_cfg = {k: 0 for k in ("fwd_warps", "fwd_bk", "bwd_a_warps", "bwd_a_bk", "bwd_r_warps", "bwd_r_bk", "bwd_dh")}
_last = {"sg_fwd": "", "sg_bwd": "", "shared_fwd": "", "shared_bwd": ""}
_enabled = [True, True]
_workspaces: dict = {}
_MAX_WORKSPACES = 8          # (device, stream) pairs kept; the least recently used buffer is dropped beyond that


def _call(fn, *args):
    status = fn(*args)
    if status != _cabi.OK:
        raise RuntimeError(_cabi.last_error())


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def _workspace(device, nbytes: int) -> torch.Tensor:
    """Scratch buffer cached per device and stream (two streams must not share one: their kernels may
    overlap).  A buffer grows on demand; at most `_MAX_WORKSPACES` are kept, least recently used first
    out, and `release_workspaces()` drops them all."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.pop(key, None)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)
    _workspaces[key] = buf                       # re-inserted last: dicts keep insertion order
    while len(_workspaces) > _MAX_WORKSPACES:
        _workspaces.pop(next(iter(_workspaces)))
    return buf


def release_workspaces() -> None:
    """Drops every cached scratch buffer (they are re-created on the next backward)."""
    _workspaces.clear()


# --------------------------------------------------------------------------- checks
# Messages follow single_gather_check / single_gather_shared_check
# (cuda/forward.cu:1609-1653) so callers' `pytest.raises(match=...)` keep working.

def _check_single(xs, mask, who="single_gather"):
    Q = xs[0]
    if not (isinstance(Q, torch.Tensor) and Q.is_cuda):
        raise RuntimeError(f"{who}: inputs must be CUDA tensors")
    if Q.dim() != 4:
        raise RuntimeError(f"{who}: inputs must be [B,H,N,D]")
    B, H, N, D = Q.shape
    if not (B > 0 and H > 0 and N > 0):
        raise RuntimeError(f"{who}: empty batch/head/sequence")
    if D not in (64, 128):
        raise RuntimeError(f"{who}: D must be 64 or 128, got {D}")
    if N % 16:
        raise RuntimeError(f"{who}: N must be a multiple of 16, got {N}")
    for x in xs:
        if not (x.is_cuda and x.device == Q.device):
            raise RuntimeError(f"{who}: all inputs must be on one CUDA device")
        if x.dtype != _BF16:
            raise RuntimeError(f"{who}: inputs must be bf16")
        if not x.is_contiguous():
            raise RuntimeError(f"{who}: inputs must be contiguous")
        if x.shape != Q.shape:
            raise RuntimeError(f"{who}: all inputs must share one shape")
    if mask is not None:
        if not (mask.is_cuda and mask.device == Q.device):
            raise RuntimeError(f"{who}: mask must be on the input device")
        if mask.dtype != torch.bool:
            raise RuntimeError(f"{who}: mask must be bool")
        if not mask.is_contiguous():
            raise RuntimeError(f"{who}: mask must be contiguous")
        if tuple(mask.shape) != (B, N, N):
            raise RuntimeError(f"{who}: mask must be [B,N,N]")


def _check_shared(Q, kv, mask, window, group, who="single_gather_shared", need_mask=True):
    if not (isinstance(Q, torch.Tensor) and Q.is_cuda and Q.dim() == 4):
        raise RuntimeError(f"{who}: Q must be a CUDA [B,Hq,N,D] tensor")
    B, H, N, D = Q.shape
    if not (B > 0 and H > 0):
        raise RuntimeError(f"{who}: empty batch/head dimensions are unsupported")
    if D != 128:
        raise RuntimeError(f"{who}: D must be 128 (prototype), got {D}")
    if not (N > 0 and N % 16 == 0):
        raise RuntimeError(f"{who}: N must be a positive multiple of 16, got {N}")
    if window not in (16, 32, 64, 128):
        raise RuntimeError(f"{who}: window must be 16, 32, 64 or 128, got {window}")
    if group not in (1, 2, 4):
        raise RuntimeError(f"{who}: head group must be 1, 2 or 4, got {group}")
    if H % group:
        raise RuntimeError(f"{who}: Hq={H} is not divisible by the head group {group}")
    if not (Q.dtype == _BF16 and Q.is_contiguous()):
        raise RuntimeError(f"{who}: Q must be contiguous bf16")
    for x in kv:
        if not (isinstance(x, torch.Tensor) and x.is_cuda and x.device == Q.device and x.dtype == _BF16
                and x.is_contiguous()):
            raise RuntimeError(f"{who}: KV tensors must be contiguous bf16 on Q's device")
        if tuple(x.shape) != (B, 1, N, D):
            raise RuntimeError(f"{who}: KV tensors must be [B,1,N,D] (Hkv = 1), got {tuple(x.shape)}")
    if mask is None and not need_mask:
        return
    if not (isinstance(mask, torch.Tensor) and mask.is_cuda and mask.device == Q.device and mask.dtype == torch.bool
            and mask.is_contiguous() and tuple(mask.shape) == (B, N, N)):
        raise RuntimeError(f"{who}: mask must be a contiguous bool [B,N,N] on Q's device (the window mask)")


def _check_state(Q, tensors, who):
    """Saved forward state must live on Q's device (cuda/backward.cu:2377-2392)."""
    for name, t, shape in tensors:
        if not (isinstance(t, torch.Tensor) and t.is_cuda and t.device == Q.device):
            raise RuntimeError(f"{who}: {name} must be on Q's device ({Q.device})")
        if not t.is_contiguous() or tuple(t.shape) != tuple(shape):
            raise RuntimeError(f"{who}: {name} must be contiguous with shape {tuple(shape)}")


# --------------------------------------------------------------------------- raw ops (mask optional)

def pack_mask(mask: torch.Tensor, window: int = 0, with_support: bool = False):
    """Bool/byte mask [B,N,N] -> packed words int32 [B,N,ceil(N/32)] (bit t of word c = key 32 c + t), restricted to
    the causal window when window > 0; with_support also returns the per-query count of visible keys saturated at
    2 ([B,N] uint8).  The packed form is what `mask_words=` of the raw calls takes."""
    B, N, _ = mask.shape
    mask = mask.contiguous()
    with torch.cuda.device(mask.device):
        words = torch.empty((B, N, (N + 31) // 32), dtype=torch.int32, device=mask.device)
        support = torch.empty((B, N), dtype=torch.uint8, device=mask.device) if with_support else None
        _call(lib.att3_sg_pack_mask, mask.data_ptr(), words.data_ptr(), _ptr(support), B, N, int(window), _stream(mask))
    return (words, support) if with_support else words


def _ext(window_s: int, mask_words, bnhd: bool = False, y_act=None, precise: bool = False):
    """att3_sg_ext for a call, or None for the plain entry points."""
    if not window_s and mask_words is None and not bnhd and y_act is None and not precise:
        return None
    return _cabi.SgExt(int(window_s), _ptr(mask_words), 1 if bnhd else 0, _ptr(y_act), 1 if precise else 0)


def _dims(Q, R, bnhd: bool):
    """(B, Hq, Hkv, N, D) of operands laid out [B,H,N,D] or, with bnhd, [B,N,H,D]."""
    if bnhd:
        B, N, Hq, D = Q.shape
        return B, Hq, R.shape[2], N, D
    B, Hq, N, D = Q.shape
    return B, Hq, R.shape[1], N, D


def sg_forward_raw(Q, R, S, Vr, Vs, mask, window: int, q_begin: int = 0, window_s: int = 0, mask_words=None,
                   bnhd: bool = False, act: bool = False, precise: bool = False):
    """Windowed/dense single gather on already-validated BF16 tensors.  mask may be
    None: with window > 0 the causal window is generated from indices inside the
    kernel, so no [B,N,N] tensor is ever materialised.  window_s > 0: another window on the
    S / Vs key axis (`window` is then the R / Vr axis's); mask_words: the mask as packed words
    (see pack_mask) instead of `mask`; bnhd: the operands (and Y) are [B,N,H,D] contiguous
    instead of [B,H,N,D]; act: also return QuickGELU(Y) as a fourth result, written by the
    forward's epilogue; precise: score products on the exact split of Q o R (value + residual), to be
    used with the same setting in the backward.  m, l are [B,H,N] either way."""
    B, Hq, Hkv, N, D = _dims(Q, R, bnhd)
    with torch.cuda.device(Q.device):
        Y = torch.empty_like(Q)
        Ya = torch.empty_like(Q) if act else None
        m = torch.empty((B, Hq, N), dtype=torch.float32, device=Q.device)
        l = torch.empty_like(m)
        ext = _ext(window_s, mask_words, bnhd, Ya, precise)
        args = (Q.data_ptr(), R.data_ptr(), S.data_ptr(), Vr.data_ptr(), Vs.data_ptr(),
                _ptr(mask), Y.data_ptr(), m.data_ptr(), l.data_ptr(), B, Hq, Hkv, N, D, int(window), int(q_begin),
                _stream(Q))
        if ext is None:
            _call(lib.att3_sg_forward, *args)
        else:
            _call(lib.att3_sg_forward_ext, *args, C.byref(ext))
    return (Y, m, l, Ya) if act else (Y, m, l)


def sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, mask, window: int, q_begin: int = 0, kv_f32: bool = False,
                    window_s: int = 0, mask_words=None, bnhd: bool = False, precise: bool = False):
    """kv_f32: leave dR, dS, dVr, dVs in FP32 (partial sums of a process that holds only part of the
    query heads of a KV head; windowed path only).  window_s, mask_words, bnhd: as in sg_forward_raw
    (with bnhd the gradients come back [B,N,H,D] too)."""
    B, Hq, Hkv, N, D = _dims(Q, R, bnhd)
    ext = _ext(window_s, mask_words, bnhd, None, precise)
    if ext is not None and kv_f32:
        raise RuntimeError("sg_backward_raw: kv_f32 and the extended options do not combine")
    with torch.cuda.device(Q.device):
        dQ = torch.zeros_like(Q) if q_begin else torch.empty_like(Q)
        dR, dS, dVr, dVs = (torch.empty_like(R, dtype=torch.float32 if kv_f32 else R.dtype) for _ in range(4))
        nbytes = lib.att3_sg_backward_workspace_bytes(B, Hq, Hkv, N, D, int(window))
        ws = _workspace(Q.device, nbytes)
        args = (dY.data_ptr(), Q.data_ptr(), R.data_ptr(), S.data_ptr(), Vr.data_ptr(),
                Vs.data_ptr(), Y.data_ptr(), m.data_ptr(), l.data_ptr(), _ptr(mask),
                dQ.data_ptr(), dR.data_ptr(), dS.data_ptr(), dVr.data_ptr(), dVs.data_ptr(),
                B, Hq, Hkv, N, D, int(window), int(q_begin), ws.data_ptr(), nbytes, _stream(Q))
        if ext is not None:
            _call(lib.att3_sg_backward_ext, *args, C.byref(ext))
        else:
            _call(lib.att3_sg_backward_kv32 if kv_f32 else lib.att3_sg_backward, *args)
    return dQ, dR, dS, dVr, dVs


def sg_backward_sides_raw(dY, Q, R, S, Vr, Vs, Y, m, l, mask, window: int, q_begin: int = 0, between=None):
    """The windowed backward with FP32 key gradients, one key side per C-ABI call.  Returns
    (dQ, kv32) with kv32 an FP32 [4,B,Hkv,N,D] tensor holding dS, dVs, dR, dVr in that order: the
    first two are complete after side 0, and `between(kv32[:2])`, if given, is called at that point
    (e.g. to start an all-reduce of them that overlaps side 1)."""
    B, Hq, N, D = Q.shape
    Hkv = R.shape[1]
    with torch.cuda.device(Q.device):
        dQ = torch.zeros_like(Q) if q_begin else torch.empty_like(Q)
        kv32 = torch.empty((4, B, Hkv, N, D), dtype=torch.float32, device=Q.device)
        nbytes = lib.att3_sg_backward_workspace_bytes(B, Hq, Hkv, N, D, int(window))
        ws = _workspace(Q.device, nbytes)
        for side in (0, 1):
            _call(lib.att3_sg_backward_kv32_side, side, dY.data_ptr(), Q.data_ptr(), R.data_ptr(), S.data_ptr(),
                  Vr.data_ptr(), Vs.data_ptr(), Y.data_ptr(), m.data_ptr(), l.data_ptr(), _ptr(mask), dQ.data_ptr(),
                  kv32[2].data_ptr(), kv32[0].data_ptr(), kv32[3].data_ptr(), kv32[1].data_ptr(),
                  B, Hq, Hkv, N, D, int(window), int(q_begin), ws.data_ptr(), nbytes, _stream(Q))
            if side == 0 and between is not None:
                between(kv32[:2])
    return dQ, kv32


def device_status(device=None) -> None:
    """Synchronises the current stream and raises if a bounded device-side wait ran out."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _call(lib.att3_device_status, torch.cuda.current_stream(dev).cuda_stream)


# --------------------------------------------------------------------------- pybind-compatible surface

def _effective_window(window: int, n: int) -> int:
    """Window the kernels are told about.  A promise wider than the sequence is
    plain causal visibility of width n; one wider than the 128 resident keys of
    the ring schedule cannot be exploited, so the dense schedule runs and the
    mask alone carries the visibility (window 0)."""
    win = min(max(int(window), 0), int(n))
    return win if win <= 128 else 0


def single_gather_forward(Q, R, S, Vr, Vs, mask=None, window=0):
    """(Y bf16 [B,H,N,D], m, l fp32 [B,H,N]); cpp/cuda_bindings.cpp:51-61."""
    _check_single([Q, R, S, Vr, Vs], mask)
    if window > 0 and mask is None:
        raise RuntimeError("single_gather: window metadata needs the mask it describes")
    win = _effective_window(window, Q.shape[2])
    out = sg_forward_raw(Q, R, S, Vr, Vs, mask, win)
    _last["sg_fwd"] = f"D={Q.shape[3]} schedule={'ring' if win else 'dense'} masked={int(mask is not None)} win={win}"
    return out


def single_gather_backward(dY, Q, R, S, Vr, Vs, Y, m, l, mask=None, window=0):
    """(dQ, dR, dS, dVr, dVs) bf16; cpp/cuda_bindings.cpp:63-73."""
    _check_single([dY, Q, R, S, Vr, Vs, Y], mask, "single_gather_backward")
    B, H, N, _ = Q.shape
    _check_state(Q, [("m", m, (B, H, N)), ("l", l, (B, H, N))], "single_gather_backward")
    if window > 0 and mask is None:
        raise RuntimeError("single_gather: window metadata needs the mask it describes")
    win = _effective_window(window, N)
    out = sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, mask, win)
    _last["sg_bwd"] = f"D={Q.shape[3]} schedule={'ring' if win else 'dense'} roles=own(S),own(R) win={win}"
    return out


def single_gather_shared_forward(Q, R, S, Vr, Vs, mask, window=128, fwd_group=1):
    """Shared-KV forward; cpp/cuda_bindings.cpp:75-79.  fwd_group is accepted for
    compatibility: one schedule serves every group value."""
    _check_shared(Q, [R, S, Vr, Vs], mask, window, 1 if fwd_group == 0 else fwd_group)
    out = sg_forward_raw(Q, R, S, Vr, Vs, mask, window)
    _last["shared_fwd"] = f"D=128 Hkv=1 fwd_group={fwd_group} win={window} implementation=sm100_ring"
    return out


def single_gather_shared_backward(dY, Q, R, S, Vr, Vs, Y, m, l, mask, window=128, rs_group=1):
    """Shared-KV backward, KV gradients reduced to [B,1,N,128]; cpp/cuda_bindings.cpp:81-86."""
    _check_shared(Q, [R, S, Vr, Vs], mask, window, 1 if rs_group == 0 else rs_group, "single_gather_shared_backward")
    B, H, N, D = Q.shape
    _check_state(Q, [("dY", dY, Q.shape), ("Y", Y, Q.shape), ("m", m, (B, H, N)), ("l", l, (B, H, N))],
                 "single_gather_shared_backward")
    out = sg_backward_raw(dY, Q, R, S, Vr, Vs, Y, m, l, mask, window)
    _last["shared_bwd"] = f"D=128 Hkv=1 rs_group={rs_group} win={window} implementation=sm100_ring"
    return out


def tc_launches():
    """Launch counters (cpp/cuda_bindings.cpp:31-41)."""
    c = [int(lib.att3_launch_count(i)) for i in range(4)]
    return {"forward": c[2], "backward": c[3], "sg_forward": c[0], "sg_backward": c[1],
            "sg_shared_forward": c[0], "sg_shared_backward": c[1]}


def sg_dispatch():
    """Last schedule chosen per entry point (cpp/cuda_bindings.cpp:42-49)."""
    return {"forward": _last["sg_fwd"], "backward": _last["sg_bwd"],
            "shared_forward": _last["shared_fwd"], "shared_backward": _last["shared_bwd"]}


def sg_set_config(cfg: dict) -> None:
    """Tile overrides of the reference kernels (cpp/cuda_bindings.cpp:88-106).  The
    sm_100a kernels have one tile shape, so values are recorded and otherwise ignored."""
    for k, v in cfg.items():
        if k not in _cfg:
            raise ValueError(f"sg_set_config: unknown key {k}")
        _cfg[k] = int(v)


def sg_get_config() -> dict:
    return dict(_cfg)


def sg_tile_ranges(N, window, a, side, bj, bk):
    """[(j0, k_lo, k_hi), ...] visited by the work item anchored at `a`
    (cpp/cuda_bindings.cpp:117-132)."""
    cap = max(1, (int(N) + int(bj) - 1) // int(bj) + 1)
    buf = (C.c_int * (3 * cap))()
    n = lib.att3_sg_tile_ranges(int(N), int(window), int(a), int(side), int(bj), int(bk), buf, cap)
    if n < 0:
        raise RuntimeError("sg_tile_ranges: bad argument")
    return [(buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]) for i in range(n)]


def tc_set_enabled(forward: bool, backward: bool):
    """Returns the previous (forward, backward) gates (cpp/cuda_bindings.cpp:134-141).
    There is no scalar fallback to switch to; the flags are kept for API parity."""
    prev = tuple(_enabled)
    _enabled[0], _enabled[1] = bool(forward), bool(backward)
    return prev


# --------------------------------------------------------------------------- three-gather hypergraph attention

_HG_NAMES = ("Q", "R", "S", "Vq_1", "Vq_2", "Vr_1", "Vr_2", "Vs_1", "Vs_2")


def _check_hg(tensors, mask, who):
    """Shape contract of the three-gather operator (cuda/forward.cu:1281-1296): Q, Vq_* are [B,H,I,D], R, Vr_*
    [B,H,J,D], S, Vs_* [B,H,K,D]; a mask needs I == J == K.  Returns (mask or None, (I, J, K))."""
    Q, R, S = tensors[0], tensors[1], tensors[2]
    if not (isinstance(Q, torch.Tensor) and Q.is_cuda and Q.dim() == 4):
        raise RuntimeError(f"{who}: inputs must be CUDA [B,H,N,D] tensors")
    B, H, I, D = Q.shape
    if D not in (16, 32, 64, 128):
        raise RuntimeError(f"{who}: head dim must be 16, 32, 64 or 128, got {D}")
    lead = {"Q": Q, "Vq_1": Q, "Vq_2": Q, "R": R, "Vr_1": R, "Vr_2": R, "S": S, "Vs_1": S, "Vs_2": S}
    for name, t in zip(_HG_NAMES, tensors):
        if not (t.is_cuda and t.device == Q.device and t.dtype == _BF16 and t.is_contiguous()):
            raise RuntimeError(f"{who}: {name} must be contiguous bf16 on Q's device")
        if t.dim() != 4 or t.shape != lead[name].shape or t.shape[0] != B or t.shape[1] != H or t.shape[3] != D:
            raise RuntimeError(f"{who}: {name} is {tuple(t.shape)}, expected {tuple(lead[name].shape)} "
                               f"(batch, heads and head dim of Q; the length of its own axis)")
    J, K = R.shape[2], S.shape[2]
    for n in (I, J, K):
        if n % 16:
            raise RuntimeError(f"{who}: N must be a multiple of 16, got {n}")
    if mask is not None and mask.numel():
        if not (I == J == K):
            raise RuntimeError(f"{who}: masked/tensor-core path requires equal shapes (I == J == K), got {(I, J, K)}")
        if not (mask.is_cuda and mask.device == Q.device and mask.dtype == torch.bool and mask.is_contiguous()
                and tuple(mask.shape) == (B, I, I)):
            raise RuntimeError(f"{who}: mask must be a contiguous bool [B,N,N] on Q's device")
        return mask, (I, J, K)
    return None, (I, J, K)


def _scatter_in_use(*tensors) -> bool:
    """True if any of the tensors has a non-zero entry (host sync, as the reference's
    `scatter_used` gate: cuda/forward.cu:1541-1542)."""
    return any(bool(t.ne(0).any().item()) for t in tensors)


def forward(Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2, dropout_rate=0.0, I_valid=-1, J_valid=-1, K_valid=-1,
            mask=None, gather_mode=0):
    """Three anchored gathers (and scatters) of one score cube; returns
    (Y_q, Y_r, Y_s, Y_q_, Y_r_, Y_s_, m_i, l_i, m_j, l_j, m_k, l_k) as the reference's
    `forward` (cpp/cuda_bindings.cpp:143-177).  dropout_rate is accepted and unused,
    as in the reference (cuda/forward.cu:1259)."""
    ts = [Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2]
    mask, (I, J, K) = _check_hg(ts, mask, "forward")
    B, H, _, D = Q.shape
    # one valid length per axis, each defaulting to the padded length (cuda/forward.cu:1300-1302)
    valid = [int(v) if 0 < int(v) <= n else n for v, n in zip((I_valid, J_valid, K_valid), (I, J, K))]
    scatter = 1 if (gather_mode == 0 and _scatter_in_use(Vq_2, Vr_2, Vs_2)) else 0
    if scatter and not (I == J == K):
        raise RuntimeError(f"forward: Scatter requires I == J == K, got {(I, J, K)}")
    with torch.cuda.device(Q.device):
        outs = [torch.empty_like(t) for t in (Q, R, S, Q, R, S)]
        stats = [torch.empty((B, H, n), dtype=torch.float32, device=Q.device) for n in (I, I, J, J, K, K)]
        _call(lib.att3_hg_forward_axes, *[t.data_ptr() for t in ts], _ptr(mask), *[o.data_ptr() for o in outs],
              *[s.data_ptr() for s in stats], B, H, I, J, K, D, *valid, int(gather_mode), scatter, _stream(Q))
    return (*outs, *stats)


def backward(grad_Y_q, grad_Y_r, grad_Y_s, grad_Y_q_, grad_Y_r_, grad_Y_s_, Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1,
             Vs_2, m_i, l_i, m_j, l_j, m_k, l_k, dropout_rate=0.0, mask=None, Y_q=None, Y_r=None, Y_s=None):
    """Nine gradients from the forward's statistics (cpp/cuda_bindings.cpp:179-233).  The
    gather outputs Y_q, Y_r, Y_s are required: the Jacobian correction is rowsum(dY o Y)."""
    ts = [Q, R, S, Vq_1, Vq_2, Vr_1, Vr_2, Vs_1, Vs_2]
    mask, (I, J, K) = _check_hg(ts, mask, "backward")
    if Y_q is None or Y_r is None or Y_s is None:
        raise RuntimeError("backward: tensor-core path unavailable without the forward outputs Y_q, Y_r, Y_s")
    B, H, _, D = Q.shape
    gs = [grad_Y_q, grad_Y_r, grad_Y_s, grad_Y_q_, grad_Y_r_, grad_Y_s_]
    for g, like in zip(gs + [Y_q, Y_r, Y_s], (Q, R, S, Q, R, S, Q, R, S)):
        if not (g.is_cuda and g.device == Q.device and g.dtype == _BF16 and g.is_contiguous() and g.shape == like.shape):
            raise RuntimeError("backward: cotangents and outputs must be contiguous bf16 on Q's device, shaped like "
                               "the tensor of their axis ([B,H,I,D], [B,H,J,D], [B,H,K,D])")
    # gather_mode 1 leaves (m = +1e30, l = 1) in the R/S statistics (cuda/forward.cu:1455-1459)
    gather_mode = 1 if bool((m_j[0, 0, 0] > 1e29).item()) else 0
    scatter = 1 if (gather_mode == 0 and _scatter_in_use(grad_Y_q_, grad_Y_r_, grad_Y_s_)) else 0
    if scatter and not (I == J == K):
        raise RuntimeError(f"backward: Scatter requires I == J == K, got {(I, J, K)}")
    with torch.cuda.device(Q.device):
        grads = [torch.empty_like(t) for t in ts]
        nbytes = lib.att3_hg_backward_axes_workspace_bytes(B, H, I, J, K, D)
        ws = _workspace(Q.device, nbytes)
        # the reference's backward takes no valid lengths: padded slots take part (cpp/cuda_bindings.cpp:179-205)
        _call(lib.att3_hg_backward_axes, *[g.data_ptr() for g in gs], *[t.data_ptr() for t in ts],
              Y_q.data_ptr(), Y_r.data_ptr(), Y_s.data_ptr(),
              m_i.data_ptr(), l_i.data_ptr(), m_j.data_ptr(), l_j.data_ptr(), m_k.data_ptr(), l_k.data_ptr(),
              _ptr(mask), *[g.data_ptr() for g in grads], B, H, I, J, K, D, 0, 0, 0, gather_mode, scatter,
              ws.data_ptr(), nbytes, _stream(Q))
    return tuple(grads)
