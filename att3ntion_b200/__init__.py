"""B200-native (sm_100a) kernels for the hypergraph-attention hot path, behind the
Python surface of ``att3ntion``: ``single_gather_attention``,
``single_gather_shared_attention`` and ``HypergraphAttention``.

Attributes resolve on first use (so ``python -m att3ntion_b200.build`` can run
before the native library exists).  Resolving any of them loads
``libatt3_b200.so``; if the library is missing that raises ImportError -- there
is no CPU or eager fallback.
"""
from importlib import import_module

_EXPORTS = {
    "single_gather_attention": "._single_gather",
    "window_mask": "._single_gather",
    "single_gather_shared_attention": "._single_gather_shared",
    "HypergraphAttention": "._autograd",
    "QuickGELU": "._autograd",
}

__all__ = sorted(_EXPORTS)


def __getattr__(name):
    target = _EXPORTS.get(name)
    if target is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(import_module(target, __name__), name)
    globals()[name] = value
    return value
