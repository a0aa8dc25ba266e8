"""ctypes binding of ``libatt3_b200.so`` (the C ABI declared in ``include/att3_b200.h``).

Nothing here computes: the functions take raw device pointers.  The library is
loaded from the package directory; if it is missing the import fails loudly
rather than falling back to anything else.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libatt3_b200.so"

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_TIMEOUT = range(6)

_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t

# name -> (restype, argtypes); mirrors include/att3_b200.h declaration by declaration
SIGNATURES = {
    "att3_last_error": (C.c_char_p, []),
    "att3_abi_version": (_i, []),
    "att3_device_status": (_i, [_vp]),
    "att3_sg_backward_workspace_bytes": (_sz, [_i] * 6),
    "att3_sg_forward": (_i, [_vp] * 9 + [_i] * 7 + [_vp]),
    "att3_sg_backward": (_i, [_vp] * 15 + [_i] * 7 + [_vp, _sz, _vp]),
    "att3_sg_backward_kv32": (_i, [_vp] * 15 + [_i] * 7 + [_vp, _sz, _vp]),
    "att3_sg_forward_ext": (_i, [_vp] * 9 + [_i] * 7 + [_vp, _vp]),
    "att3_sg_backward_ext": (_i, [_vp] * 15 + [_i] * 7 + [_vp, _sz, _vp, _vp]),
    "att3_sg_pack_mask": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "att3_sg_backward_kv32_side": (_i, [_i] + [_vp] * 15 + [_i] * 7 + [_vp, _sz, _vp]),
    "att3_sg_backward_static_max_bytes": (_sz, []),
    "att3_sg_backward_static": (_i, [_vp] * 15 + [_i] * 7 + [_vp]),
    "att3_hg_forward": (_i, [_vp] * 22 + [_i] * 7 + [_vp]),
    "att3_hg_backward_workspace_bytes": (_sz, [_i] * 4),
    "att3_hg_backward": (_i, [_vp] * 34 + [_i] * 7 + [_vp, _sz, _vp]),
    "att3_hg_forward_axes": (_i, [_vp] * 22 + [_i] * 11 + [_vp]),
    "att3_hg_backward_axes_workspace_bytes": (_sz, [_i] * 6),
    "att3_hg_backward_axes": (_i, [_vp] * 34 + [_i] * 11 + [_vp, _sz, _vp]),
    "att3_sg_tile_ranges": (_i, [_i] * 6 + [C.POINTER(_i), _i]),
    "att3_pack_mask32": (C.c_uint32, [_vp, _i]),
    "att3_sg_query_blocks": (_i, [_i] * 6 + [C.POINTER(_i)]),
    "att3_sg_set_query_block": (_i, [_i, _i]),
    "att3_sg_set_packed": (_i, [_i]),
    "att3_launch_count": (C.c_ulonglong, [_i]),
    "att3_timing_enable": (_i, [_i]),
    "att3_timing_read": (_i, [_i, C.POINTER(C.c_double), C.POINTER(C.c_ulonglong)]),
    "att3_umma_selftest": (_i, [_vp, _vp, _vp, _i, _vp, _vp]),
    "att3_wait_selftest": (_i, [C.c_uint, _vp]),
}


class SgExt(C.Structure):
    """att3_sg_ext of include/att3_b200.h."""
    _fields_ = [("window_s", C.c_int), ("mask_words", C.c_void_p), ("layout", C.c_int), ("Y_act", C.c_void_p), ("precise", C.c_int)]


class Att3Error(RuntimeError):
    """Raised when a C-ABI call returns a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


def _load() -> C.CDLL:
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python -m att3ntion_b200.build` "
            "(the sm_100a kernels have no fallback path)"
        )
    lib = C.CDLL(str(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    return lib.att3_last_error().decode()


def check(status: int) -> None:
    if status != OK:
        raise Att3Error(status, last_error())
