"""All-gather -> GEMM and GEMM -> reduce-scatter as single kernels over symmetric (peer-mapped) memory.
``available`` gates on the symmetric-memory runtime being initialised for the group."""
from __future__ import annotations

_impl = None


def _load():
    global _impl
    if _impl is None:
        try:
            from . import fused_linear_impl as impl
            _impl = impl
        except ImportError:
            _impl = False
    return _impl


def available(x, weight, group=None) -> bool:
    impl = _load()
    return bool(impl) and impl.available(x, weight, group)


def allgather_linear(x, weight, group):
    return _load().allgather_linear(x, weight, group)


def linear_reduce_scatter(x, weight, group):
    return _load().linear_reduce_scatter(x, weight, group)
