"""Gradient bucketing for data parallelism (``Eager_AssignGroupBySize``,
paddle/fluid/distributed/collective/reducer.cc:48): parameters are walked in reverse creation order
(gradients become ready roughly in that order), grouped per dtype, and a group is closed when it
reaches its size limit; the first limit applies to the first group only (small, so communication starts
early), the last limit to all later groups.  The native runtime provides the same routine
(``pd_assign_group_by_size``); this module calls it when the library is built."""
from __future__ import annotations

import ctypes


def assign_group_by_size(params, group_size_limits, is_sparse=None):
    sizes = [p.numel() * p.element_size() for p in params]
    dtypes = [str(p.dtype) for p in params]
    try:
        from ..ops import _lib
        rt = _lib.runtime()
        if hasattr(rt, "pd_assign_group_by_size"):
            n = len(params)
            order = list(range(n - 1, -1, -1))
            dt_ids = {d: i for i, d in enumerate(sorted(set(dtypes)))}
            c_sizes = (ctypes.c_int64 * n)(*[sizes[i] for i in order])
            c_dt = (ctypes.c_int * n)(*[dt_ids[dtypes[i]] for i in order])
            c_lim = (ctypes.c_int64 * len(group_size_limits))(*group_size_limits)
            out = (ctypes.c_int * n)()
            ng = rt.pd_assign_group_by_size(c_sizes, c_dt, n, c_lim, len(group_size_limits), out)
            groups = [[] for _ in range(ng)]
            for k in range(n):
                groups[out[k]].append(order[k])
            return groups
    except Exception:  # noqa: BLE001 - the pure-Python routine below is the same algorithm
        pass
    groups, open_groups, limit_idx = [], {}, {}
    for i in range(len(params) - 1, -1, -1):
        d = dtypes[i]
        cur = open_groups.setdefault(d, {"idx": [], "bytes": 0})
        cur["idx"].append(i)
        cur["bytes"] += sizes[i]
        li = limit_idx.get(d, 0)
        if cur["bytes"] >= group_size_limits[min(li, len(group_size_limits) - 1)]:
            groups.append(cur["idx"])
            open_groups[d] = {"idx": [], "bytes": 0}
            limit_idx[d] = li + 1
    for cur in open_groups.values():
        if cur["idx"]:
            groups.append(cur["idx"])
    return groups
