"""Algebra on lists of half-open time ranges ``(start, end)`` (python/paddle/profiler/statistic_helper.py:17-220),
used to compute busy time, and the overlap of communication with computation, from device timelines."""
from __future__ import annotations


def merge_self_ranges(src_ranges, is_sorted=False):
    """Union of possibly overlapping ranges as a sorted list of disjoint ranges."""
    rs = list(src_ranges) if is_sorted else sorted(src_ranges)
    out = []
    for s, e in rs:
        if e <= s:
            continue
        if out and s <= out[-1][1]:
            if e > out[-1][1]:
                out[-1] = (out[-1][0], e)
        else:
            out.append((s, e))
    return out


def sum_ranges(ranges):
    return sum(e - s for s, e in ranges)


def merge_ranges(range_list1, range_list2, is_sorted=False):
    """Union of two range lists."""
    return merge_self_ranges(list(range_list1) + list(range_list2), False)


def intersection_ranges(range_list1, range_list2, is_sorted=False):
    """Time covered by both lists (each is first reduced to disjoint ranges)."""
    a, b = merge_self_ranges(range_list1, is_sorted), merge_self_ranges(range_list2, is_sorted)
    out, i, j = [], 0, 0
    while i < len(a) and j < len(b):
        s, e = max(a[i][0], b[j][0]), min(a[i][1], b[j][1])
        if s < e:
            out.append((s, e))
        if a[i][1] <= b[j][1]:
            i += 1
        else:
            j += 1
    return out


def subtract_ranges(range_list1, range_list2, is_sorted=False):
    """Time covered by the first list and not by the second."""
    a, b = merge_self_ranges(range_list1, is_sorted), merge_self_ranges(range_list2, is_sorted)
    out, j = [], 0
    for s, e in a:
        cur = s
        while j < len(b) and b[j][1] <= cur:
            j += 1
        k = j
        while k < len(b) and b[k][0] < e:
            if b[k][0] > cur:
                out.append((cur, b[k][0]))
            cur = max(cur, b[k][1])
            k += 1
        if cur < e:
            out.append((cur, e))
    return out
