"""``RecordEvent`` ranges and helpers (python/paddle/profiler/utils.py:47-260)."""
from __future__ import annotations

import functools
import json
from contextlib import ContextDecorator

import torch

from .profiler_statistic import TracerEventType, register_user_range

_is_profiler_used = False
_has_optimizer_wrapped = False


def in_profiler_mode():
    return _is_profiler_used


def _set_profiler_mode(on):
    global _is_profiler_used
    _is_profiler_used = bool(on)


class RecordEvent(ContextDecorator):
    """User range: context manager, decorator, or ``begin()`` / ``end()``.  Recorded by the activity tracer under its
    name and typed ``event_type`` in the summaries; with a GPU it also opens an NVTX range so that external timelines
    show the same names.  Outside a running profiler only the NVTX range is emitted (when a GPU is present)."""

    def __init__(self, name, event_type=TracerEventType.PythonUserDefined):
        self.name = name
        self.event_type = event_type
        self._rf = None
        self._nvtx = False

    def begin(self):
        if self.event_type is not None:
            register_user_range(self.name, self.event_type)
        if in_profiler_mode():
            self._rf = torch.profiler.record_function(self.name)
            self._rf.__enter__()
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
            self._nvtx = True

    def end(self):
        if self._nvtx:
            torch.cuda.nvtx.range_pop()
            self._nvtx = False
        if self._rf is not None:
            self._rf.__exit__(None, None, None)
            self._rf = None

    def __enter__(self):
        self.begin()
        return self

    def __exit__(self, *exc):
        self.end()
        return False


def load_profiler_result(filename):
    """A saved chrome trace back as a ``ProfilerResult`` whose statistics can be tabulated again."""
    from .profiler import ProfilerResult
    with open(filename) as f:
        return ProfilerResult.from_chrome_trace(json.load(f))


def wrap_optimizers():
    """Put every optimizer's ``step`` under an ``Optimization`` range so that the model view can attribute it."""
    global _has_optimizer_wrapped
    if _has_optimizer_wrapped:
        return
    from .. import optimizer as opt_mod

    def wrap(cls):
        orig = cls.__dict__.get("step")
        if orig is None or getattr(orig, "_profiler_wrapped", False):
            return

        @functools.wraps(orig)
        def step(self, *a, **k):
            if not in_profiler_mode():
                return orig(self, *a, **k)
            with RecordEvent("Optimizer.step#" + type(self).__name__, TracerEventType.Optimization):
                return orig(self, *a, **k)
        step._profiler_wrapped = True
        cls.step = step
    for name in dir(opt_mod):
        obj = getattr(opt_mod, name)
        if isinstance(obj, type) and hasattr(obj, "step"):
            wrap(obj)
    _has_optimizer_wrapped = True


def job_schedule_profiler_range(iter_id, start, end, exit_after_prof=True):
    """True while ``start <= iter_id < end``: a training loop brackets those iterations for an external timeline tool
    (the CUDA profiler API is started at ``start`` and stopped at ``end``); with ``exit_after_prof`` the process ends
    once the window has been recorded."""
    import sys
    if start < 0 or end <= start:
        return False
    if iter_id == start and torch.cuda.is_available():
        torch.cuda.profiler.start()
    if iter_id >= end:
        if torch.cuda.is_available():
            torch.cuda.profiler.stop()
        if exit_after_prof:
            sys.exit(0)
        return False
    return iter_id >= start


_nvprof_range = job_schedule_profiler_range
_job_schedule_profiler = False


def switch_job_schedule_profiler(model=None, iter_id=0, start=-1, end=-1, exit_after_prof=True):
    global _job_schedule_profiler
    _job_schedule_profiler = job_schedule_profiler_range(iter_id, start, end, exit_after_prof)
    return _job_schedule_profiler
