"""Recompute for hybrid (tensor-parallel) training: the saved inputs of a recompute block are partitioned over the
model-parallel group and/or moved to pinned host memory, and put back together when backward re-runs the block
(python/paddle/distributed/fleet/recompute/recompute_hybrid.py:48 ``_split_activation``, :69 ``_merge_activation``,
:84 ``_HPRecomputeFunction``, :265 ``recompute_hybrid``).

The autograd function that does the work is the package's :class:`RecomputeFunction` (it takes the partition
group and the offload switch as arguments); this module supplies the activation split / merge helpers and the
public entry point with the reference's ``ctx`` dictionary.
"""
from __future__ import annotations

import torch

from ...._core.tensor import as_tensor
from . import RecomputeFunction as _HPRecomputeFunction  # noqa: F401  (same class, reference name)
from . import recompute as _recompute

__all__ = []


def _split_activation(tensor, mp_group):
    """This rank's 1/mp_degree slice of the flattened activation (a copy, so the full tensor can be freed)."""
    n = mp_group.nranks
    if n < 2:
        return tensor
    numel = tensor.numel()
    assert numel != 0, "can't recompute zero element"
    assert numel % n == 0, f"The capacity of the activation ({numel}) cannot be divisible by mp_degree({n})"
    per = numel // n
    start = mp_group.rank * per
    return as_tensor(tensor.detach().reshape(-1)[start:start + per].clone())


def _merge_activation(tensor, mp_group):
    """Inverse of :func:`_split_activation`: all-gather the slices of every model-parallel rank (flat result)."""
    n = mp_group.nranks
    if n < 2:
        return tensor
    from ... import collective as C
    parts = []
    C.all_gather(parts, tensor, mp_group)
    return as_tensor(torch.cat([p.reshape(-1) for p in parts]))


def recompute_hybrid(ctx, function, *args, **kwargs):
    """Recompute ``function(*args, **kwargs)`` in backward.

    ``ctx`` keys: ``mp_group`` (required), ``offload`` (saved inputs go to pinned host memory), ``partition`` (saved
    inputs are split over ``mp_group`` and all-gathered on use), ``preserve_rng_state``."""
    mp_group = ctx.get("mp_group", None)
    assert mp_group is not None, "ctx must contains mp_group and mp_group can not be None."
    return _recompute(function, *args, offload=ctx.get("offload", False),
                      _partition_group=mp_group if ctx.get("partition", False) else None,
                      preserve_rng_state=ctx.get("preserve_rng_state", True), **kwargs)


class _CallableModule(type(__import__("sys"))):
    """The package exports a function with this module's name; whichever of the two a caller ends up holding,
    calling it runs :func:`recompute_hybrid`."""

    def __call__(self, ctx, function, *args, **kwargs):
        return recompute_hybrid(ctx, function, *args, **kwargs)


__import__("sys").modules[__name__].__class__ = _CallableModule
