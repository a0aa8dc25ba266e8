"""CPU-side checks of the C ABI: the library loads, exports every function the
public header declares, rejects bad arguments before touching a device, and its
host helpers agree with the reference's tile-range and mask-packing contract."""
import ctypes as C
import json
import re

import numpy as np
import pytest

from conftest import GOLDEN, REPO
from att3ntion_b200 import _cabi, _cuda_kernels as ck

HEADER = (REPO / "include" / "att3_b200.h").read_text()


def declared_functions():
    body = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(att3_[a-z0-9_]+)\s*\(", body)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 14
    for n in names:
        assert hasattr(_cabi.lib, n), f"{n} declared in include/att3_b200.h but not exported"
        assert n in _cabi.SIGNATURES, f"{n} has no ctypes signature in _cabi.py"


def test_abi_version_and_error_text():
    assert _cabi.lib.att3_abi_version() == 2
    rc = _cabi.lib.att3_sg_forward(None, None, None, None, None, None, None, None, None, 1, 2, 1, 24, 128, 128, 0, None)
    assert rc == _cabi.ERR_INVALID and "multiple of 16" in _cabi.last_error()
    rc = _cabi.lib.att3_sg_forward(None, None, None, None, None, None, None, None, None, 0, 2, 1, 32, 128, 128, 0, None)
    assert rc == _cabi.ERR_INVALID and "empty batch/head" in _cabi.last_error()
    rc = _cabi.lib.att3_sg_forward(None, None, None, None, None, None, None, None, None, 1, 3, 2, 32, 128, 128, 0, None)
    assert rc == _cabi.ERR_INVALID and "divisible" in _cabi.last_error()
    rc = _cabi.lib.att3_sg_forward(None, None, None, None, None, None, None, None, None, 1, 2, 1, 32, 96, 128, 0, None)
    assert rc == _cabi.ERR_INVALID and "D must be 64 or 128" in _cabi.last_error()
    rc = _cabi.lib.att3_sg_forward(None, None, None, None, None, None, None, None, None, 1, 2, 1, 32, 128, 128, 0, None)
    assert rc == _cabi.ERR_INVALID and "null" in _cabi.last_error()


def test_workspace_size_formula():
    """Two key gradients x P partial planes of [B,Hkv,N,D] floats, plus delta [B,Hq,N] floats.  P follows from the
    backward's query-block length: blocks of at least 127 queries need 2 planes, shorter blocks more."""
    lib = _cabi.lib
    n = lib.att3_sg_backward_workspace_bytes(4, 8, 1, 8192, 128, 128)
    assert n == 2 * 2 * 4 * 1 * 8192 * 128 * 4 + 4 * 8 * 8192 * 4        # 148 SMs / 4 batches: 222 queries per block
    # one short sequence: 148 blocks of 16 queries -> ceil(127 / 16) + 1 = 9 planes
    n = lib.att3_sg_backward_workspace_bytes(1, 4, 1, 1024, 128, 64)
    assert n == 2 * 9 * 1 * 1 * 1024 * 128 * 4 + 1 * 4 * 1024 * 4
    assert lib.att3_sg_set_query_block(0, 64) == _cabi.OK                # forced block length: ceil(127 / 64) + 1 = 3
    try:
        assert lib.att3_sg_backward_workspace_bytes(4, 8, 1, 8192, 128, 128) == 2 * 3 * 4 * 8192 * 128 * 4 + 4 * 8 * 8192 * 4
    finally:
        lib.att3_sg_set_query_block(0, 0)
    assert lib.att3_sg_set_query_block(8, 0) == _cabi.ERR_INVALID


def test_query_block_partition():
    blk = C.c_int(0)
    ctas = _cabi.lib.att3_sg_query_blocks(4, 8, 1, 8192, 0, 148, C.byref(blk))
    assert ctas <= 148 and ctas % 4 == 0          # one CTA per SM
    assert blk.value * (ctas // 4) >= 8192 > blk.value * (ctas // 4 - 1)


with open(GOLDEN / "bounds.json") as f:
    BOUNDS = json.load(f)


def test_tile_ranges_match_reference_bounds():
    assert len(BOUNDS["ranges"]) > 1000
    for r in BOUNDS["ranges"]:
        got = ck.sg_tile_ranges(r["N"], r["w"], r["a"], r["side"], r["bj"], r["bk"])
        assert got == [tuple(b) for b in r["blocks"]], r


def test_tile_ranges_cover_every_visible_pair_once():
    # exact single coverage and no broadening by padding (the property the reference's host test demands)
    for N, w in [(33, 7), (64, 16), (65, 32), (129, 1), (96, 40)]:
        for bj, bk in [(32, 16), (64, 32)]:
            for a in range(N):
                seen = np.zeros((N + bj, N + bk), dtype=np.int32)
                for j0, kl, kh in ck.sg_tile_ranges(N, w, a, 0, bj, bk):
                    assert (kh - kl) % bk == 0
                    seen[j0:j0 + bj, kl:kh] += 1
                lo = max(a - w + 1, 0)
                assert (seen[lo:a + 1, lo:a + 1] == 1).all()
                assert seen.max() <= 1


def test_pack_mask32_matches_reference():
    assert len(BOUNDS["pack"]) > 700
    for case in BOUNDS["pack"]:
        buf = np.zeros(case["offset"] + case["lim"] + 8, dtype=np.uint8)
        base = buf.ctypes.data
        shift = (-base) % 8                      # an 8-byte aligned origin, then the recorded misalignment
        row = buf[shift + case["offset"]: shift + case["offset"] + case["lim"]]
        row[:] = case["bytes"]
        got = _cabi.lib.att3_pack_mask32(C.c_void_p(base + shift + case["offset"]), case["lim"])
        assert got == case["word"], case


def test_shim_rejections_need_no_gpu():
    import torch
    x = torch.zeros(1, 2, 32, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        ck.single_gather_forward(x, x, x, x, x)
    with pytest.raises(RuntimeError, match="Q must be a CUDA"):
        ck.single_gather_shared_forward(x, x, x, x, x, None)
    with pytest.raises(ValueError, match="unknown key"):
        ck.sg_set_config({"nonsense": 1})
    ck.sg_set_config({"fwd_warps": 4})
    assert ck.sg_get_config()["fwd_warps"] == 4
    ck.sg_set_config({"fwd_warps": 0})
    assert ck.tc_set_enabled(True, True) == (True, True)
    assert set(ck.tc_launches()) >= {"forward", "backward", "sg_forward", "sg_backward"}


def test_three_gather_axes_are_checked_before_any_device_work():
    """Per-axis lengths of the three-gather operator: every axis a multiple of 16, a mask and the scatter outputs
    only with I == J == K (the reference's checks, cuda/forward.cu:1292, 1545)."""
    lib = _cabi.lib
    nul = [None] * 22
    one = C.c_void_p(16)          # a non-null mask pointer; the call is rejected before anything reads it

    def fwd(mask, I, J, K, scatter=0, D=64):
        args = list(nul)
        args[9] = mask
        return lib.att3_hg_forward_axes(*args, 1, 1, I, J, K, D, 0, 0, 0, 0, scatter, None)

    assert fwd(None, 32, 40, 32) == _cabi.ERR_INVALID and "multiple of 16" in _cabi.last_error()
    assert fwd(one, 32, 48, 32) == _cabi.ERR_INVALID and "mask requires I == J == K" in _cabi.last_error()
    assert fwd(None, 32, 48, 32, scatter=1) == _cabi.ERR_INVALID and "scatter requires I == J == K" in _cabi.last_error()
    assert fwd(None, 32, 48, 64, D=48) == _cabi.ERR_INVALID and "head dim" in _cabi.last_error()
    assert fwd(None, 32, 48, 64) == _cabi.ERR_INVALID and "null" in _cabi.last_error()
    # workspace: planes sized for the longest axis
    n = lib.att3_hg_backward_axes_workspace_bytes(2, 2, 32, 160, 48, 64)
    assert n == lib.att3_hg_backward_workspace_bytes(2, 2, 160, 64) > 0
