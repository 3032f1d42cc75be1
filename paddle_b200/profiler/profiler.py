"""``paddle.profiler`` (python/paddle/profiler/profiler.py:358): scheduler states CLOSED / READY / RECORD /
RECORD_AND_RETURN driven by ``step()``, targets, ``export_chrome_tracing``, ``summary`` tables and the
reader-cost / batch-cost / ips timer (profiler/timer.py).  Events come from torch.profiler (Kineto/CUPTI);
``RecordEvent`` also emits an NVTX range so external timelines see the same names."""
from __future__ import annotations

import enum
import os
import time

import torch

from .profiler_statistic import (SortedKeys, StatisticData, SummaryView, _build_table, chrome_trace_of,  # noqa: F401
                                 events_from_chrome_trace)
from .timer import benchmark
from .utils import RecordEvent, _set_profiler_mode, wrap_optimizers  # noqa: F401


class ProfilerState(enum.Enum):
    CLOSED = 0
    READY = 1
    RECORD = 2
    RECORD_AND_RETURN = 3


class ProfilerTarget(enum.Enum):
    CPU = 0
    GPU = 1
    XPU = 2
    CUSTOM_DEVICE = 3


def make_scheduler(*, closed, ready, record, repeat=0, skip_first=0):
    """step -> state (profiler.py:129-217)."""
    period = closed + ready + record

    def sched(step):
        if step < skip_first:
            return ProfilerState.CLOSED
        step -= skip_first
        if repeat > 0 and step // period >= repeat:
            return ProfilerState.CLOSED
        m = step % period
        if m < closed:
            return ProfilerState.CLOSED
        if m < closed + ready:
            return ProfilerState.READY
        if m < period - 1:
            return ProfilerState.RECORD
        return ProfilerState.RECORD_AND_RETURN
    return sched


def _default_scheduler(step):
    return ProfilerState.RECORD


def export_chrome_tracing(dir_name, worker_name=None):
    os.makedirs(dir_name, exist_ok=True)

    def handler(prof):
        name = worker_name or f"host_{os.uname().nodename}pid_{os.getpid()}"
        prof.export(os.path.join(dir_name, f"{name}_time_{int(time.time() * 1000)}.paddle_trace.json"), "json")
    return handler


def export_protobuf(dir_name, worker_name=None):
    return export_chrome_tracing(dir_name, worker_name)


class ProfilerResult:
    """Events of one recording window with their statistics; what ``load_profiler_result`` returns."""

    def __init__(self, host_events, mem_events=(), chrome_trace=None):
        self.host_events, self.mem_events, self.chrome_trace = list(host_events), list(mem_events), chrome_trace
        self._stats = None

    @classmethod
    def from_chrome_trace(cls, doc):
        host, mem = events_from_chrome_trace(doc)
        return cls(host, mem, doc)

    def get_data(self):
        return self.host_events

    @property
    def statistic_data(self):
        if self._stats is None:
            self._stats = StatisticData(self.host_events, self.mem_events)
        return self._stats

    def summary(self, sorted_by=SortedKeys.CPUTotal, op_detail=True, thread_sep=False, time_unit="ms", views=None, row_limit=100):
        return _build_table(self.statistic_data, sorted_by, op_detail, thread_sep, time_unit, row_limit, views=views)

    def save(self, path, format="json"):
        import json
        with open(path, "w") as f:
            json.dump(self.chrome_trace or {"traceEvents": []}, f)


def _get_supported_targets():
    return [ProfilerTarget.CPU] + ([ProfilerTarget.GPU] if torch.cuda.is_available() else [])


class Profiler:
    def __init__(self, *, targets=None, scheduler=None, on_trace_ready=None, record_shapes=False, profile_memory=False,
                 timer_only=False, emit_nvtx=False, custom_device_types=None, with_flops=False):
        self.targets = [t for t in (targets or _get_supported_targets()) if t in _get_supported_targets()] or [ProfilerTarget.CPU]
        if isinstance(scheduler, (tuple, list)):
            lo, hi = scheduler
            scheduler = make_scheduler(closed=max(lo - 1, 0), ready=1 if lo > 0 else 0, record=hi - lo, repeat=1)
        self.scheduler = scheduler or _default_scheduler
        self.on_trace_ready = on_trace_ready
        self.record_shapes, self.profile_memory, self.timer_only = record_shapes, profile_memory, timer_only
        self.step_num = 0
        self.current_state = ProfilerState.CLOSED
        self._prof = None
        self._last = None
        self.emit_nvtx, self.with_flops = emit_nvtx, with_flops
        self.profiler_result = None
        self._step_range = None
        if not timer_only:
            wrap_optimizers()

    def _activities(self):
        acts = [torch.profiler.ProfilerActivity.CPU]
        if ProfilerTarget.GPU in self.targets and torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        return acts

    def _open(self):
        if self.timer_only or self._prof is not None:
            return
        self._prof = torch.profiler.profile(activities=self._activities(), record_shapes=self.record_shapes,
                                            profile_memory=self.profile_memory, with_flops=self.with_flops)
        self._prof.__enter__()
        _set_profiler_mode(True)
        self._open_step_range()

    def _close(self, ret):
        if self._prof is None:
            return
        self._close_step_range()
        _set_profiler_mode(False)
        self._prof.__exit__(None, None, None)
        self._last, self._prof = self._prof, None
        self.profiler_result = None
        self._result()                       # the tracer lets a window be written once: read it now, keep the events
        if ret and self.on_trace_ready is not None:
            self.on_trace_ready(self)

    def _open_step_range(self):
        if self._prof is not None and self._step_range is None:
            self._step_range = torch.profiler.record_function(f"ProfileStep#{self.step_num}")
            self._step_range.__enter__()

    def _close_step_range(self):
        if self._step_range is not None:
            self._step_range.__exit__(None, None, None)
            self._step_range = None

    def start(self):
        benchmark().begin()
        self.current_state = self.scheduler(self.step_num)
        if self.current_state in (ProfilerState.RECORD, ProfilerState.RECORD_AND_RETURN):
            self._open()

    def stop(self):
        benchmark().end()
        self._close(self.current_state in (ProfilerState.RECORD, ProfilerState.RECORD_AND_RETURN))
        self.current_state = ProfilerState.CLOSED

    def step(self, num_samples=None):
        benchmark().step(num_samples)
        self._close_step_range()
        prev = self.current_state
        self.step_num += 1
        self.current_state = self.scheduler(self.step_num)
        recording = (ProfilerState.RECORD, ProfilerState.RECORD_AND_RETURN)
        if prev in recording and (prev == ProfilerState.RECORD_AND_RETURN or self.current_state not in recording):
            self._close(True)
        if self.current_state in recording:
            self._open()
            self._open_step_range()

    def step_info(self, unit=None):
        """``reader_cost: .. s batch_cost: .. s ips: .. <unit>/s`` averaged since the previous call."""
        return benchmark().step_info(unit)

    def _result(self):
        p = self._last or self._prof
        if p is None:
            return None
        if self.profiler_result is None:
            self.profiler_result = ProfilerResult.from_chrome_trace(chrome_trace_of(p))
        return self.profiler_result

    def export(self, path="", format="json"):
        """Write the last recording window as a chrome trace (loadable in Perfetto / chrome://tracing)."""
        res = self._result()
        if res is not None:
            res.save(path, format)

    def summary(self, sorted_by=SortedKeys.CPUTotal, op_detail=True, thread_sep=False, time_unit="ms", views=None, row_limit=100):
        """Print (and return) the statistic tables of the last recording window; ``views`` picks some of them."""
        res = self._result()
        if res is None:
            print("no profile data")
            return ""
        table = res.summary(sorted_by, op_detail, thread_sep, time_unit, views, row_limit)
        print(table)
        return table

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *a):
        self.stop()


def get_profiler(config_path):
    """A ``Profiler`` described by a JSON file: ``{"targets": ["CPU", "GPU"], "scheduler": [start, end] or
    {"closed": .., "ready": .., "record": .., "repeat": ..}, "on_trace_ready": {"export_chrome_tracing": {"dir_name": ..}},
    "timer_only": false, "record_shapes": .., "profile_memory": ..}``; a missing file gives the default profiler."""
    import json
    try:
        with open(config_path) as f:
            cfg = json.load(f)
    except (OSError, ValueError):
        return Profiler()
    kw = {}
    if "targets" in cfg:
        kw["targets"] = [ProfilerTarget[t.upper()] for t in cfg["targets"] if t.upper() in ProfilerTarget.__members__]
    sch = cfg.get("scheduler")
    if isinstance(sch, (list, tuple)):
        kw["scheduler"] = tuple(sch)
    elif isinstance(sch, dict):
        kw["scheduler"] = make_scheduler(**sch.get("make_scheduler", sch))
    otr = cfg.get("on_trace_ready")
    if isinstance(otr, dict):
        for fn_name, fn_kw in otr.items():
            fn = {"export_chrome_tracing": export_chrome_tracing, "export_protobuf": export_protobuf}.get(fn_name)
            if fn is not None:
                kw["on_trace_ready"] = fn(**fn_kw)
    for k in ("timer_only", "record_shapes", "profile_memory", "with_flops", "emit_nvtx"):
        if k in cfg:
            kw[k] = cfg[k]
    return Profiler(**kw)
