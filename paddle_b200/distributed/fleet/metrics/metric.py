"""Distributed metric reductions (python/paddle/distributed/fleet/metrics/metric.py): each function takes the local
statistic (tensor, ndarray or number), all-reduces it over the workers through ``fleet.util`` and returns the global
value as a NumPy value."""
from __future__ import annotations

import builtins

import numpy as np


def _np(x):
    if hasattr(x, "numpy"):
        return np.asarray(x.numpy())
    return np.asarray(x)


def _util(util):
    if util is not None:
        return util
    from .. import util as fleet_util
    return fleet_util


def sum(input, scope=None, util=None):                       # noqa: A001
    return _util(util).all_reduce(_np(input), "sum")


def max(input, scope=None, util=None):                       # noqa: A001
    return _util(util).all_reduce(_np(input), "max")


def min(input, scope=None, util=None):                       # noqa: A001
    return _util(util).all_reduce(_np(input), "min")


def auc(stat_pos, stat_neg, scope=None, util=None):
    """Global AUC from per-worker histograms of positive / negative counts per score bucket."""
    pos = _util(util).all_reduce(_np(stat_pos).astype(np.float64), "sum").reshape(-1)
    neg = _util(util).all_reduce(_np(stat_neg).astype(np.float64), "sum").reshape(-1)
    area, tot_pos, tot_neg = 0.0, 0.0, 0.0
    for i in range(len(pos) - 1, -1, -1):                    # from the highest score bucket down
        new_pos, new_neg = tot_pos + pos[i], tot_neg + neg[i]
        area += (new_neg - tot_neg) * (tot_pos + new_pos) / 2.0
        tot_pos, tot_neg = new_pos, new_neg
    if tot_pos * tot_neg == 0:
        return 0.5
    return float(area / (tot_pos * tot_neg))


def mae(abserr, total_ins_num, scope=None, util=None):
    e = _util(util).all_reduce(_np(abserr).astype(np.float64), "sum")
    n = _util(util).all_reduce(_np(total_ins_num).astype(np.float64), "sum")
    return float(np.sum(e) / builtins.max(float(np.sum(n)), 1.0))


def mse(sqrerr, total_ins_num, scope=None, util=None):
    e = _util(util).all_reduce(_np(sqrerr).astype(np.float64), "sum")
    n = _util(util).all_reduce(_np(total_ins_num).astype(np.float64), "sum")
    return float(np.sum(e) / builtins.max(float(np.sum(n)), 1.0))


def rmse(sqrerr, total_ins_num, scope=None, util=None):
    return float(np.sqrt(mse(sqrerr, total_ins_num, scope, util)))


def acc(correct, total, scope=None, util=None):
    c = _util(util).all_reduce(_np(correct).astype(np.float64), "sum")
    t = _util(util).all_reduce(_np(total).astype(np.float64), "sum")
    return float(np.sum(c) / builtins.max(float(np.sum(t)), 1.0))
