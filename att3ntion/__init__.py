"""The reference's import name, served by the sm_100a implementation.

A caller written against the reference package keeps its imports:

    from att3ntion import HypergraphAttention, single_gather_attention, single_gather_shared_attention
    from att3ntion import _cuda_kernels as ck          # the binding-level functions, same names

Everything here is an alias of ``att3ntion_b200``; importing this package loads
``libatt3_b200.so`` and fails with ImportError if it is missing (the reference's
package fails the same way without its compiled extension).  The reference's naive
O(N^3)-memory modules (``_HypergraphAttentionNaive``, ``PolyAttention``, ...) are
CPU baselines outside the kernel path and are not provided.
"""
import sys
from importlib import import_module

for _name in ("_cuda_kernels", "_autograd", "_custom_op", "_single_gather", "_single_gather_shared"):
    _mod = import_module(f"att3ntion_b200.{_name}")
    sys.modules[f"{__name__}.{_name}"] = _mod
    globals()[_name] = _mod

from att3ntion_b200 import (  # noqa: E402
    HypergraphAttention,
    QuickGELU,
    single_gather_attention,
    single_gather_shared_attention,
    window_mask,
)

__all__ = ["HypergraphAttention", "QuickGELU", "single_gather_attention", "single_gather_shared_attention",
           "window_mask"]
