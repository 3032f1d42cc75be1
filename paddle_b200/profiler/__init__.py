"""``paddle.profiler`` (python/paddle/profiler/profiler.py:358): scheduler states CLOSED / READY / RECORD /
RECORD_AND_RETURN driven by ``step()``, targets, ``export_chrome_tracing``, ``summary`` tables and the
reader-cost / batch-cost / ips timer (profiler/timer.py).  Events come from torch.profiler (Kineto/CUPTI);
``RecordEvent`` also emits an NVTX range so external timelines see the same names."""
from __future__ import annotations

import enum
import os
import time

import torch


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


class SummaryView(enum.Enum):
    DeviceView = 0
    OverView = 1
    ModelView = 2
    DistributedView = 3
    KernelView = 4
    OperatorView = 5
    MemoryView = 6
    MemoryManipulationView = 7
    UDFView = 8


class SortedKeys(enum.Enum):
    CPUTotal = 0
    CPUAvg = 1
    CPUMax = 2
    CPUMin = 3
    GPUTotal = 4
    GPUAvg = 5
    GPUMax = 6
    GPUMin = 7


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


class RecordEvent:
    """User range: context manager or begin()/end() (python/paddle/profiler/utils.py:47)."""

    def __init__(self, name, event_type=None):
        self.name = name
        self._rf = None

    def begin(self):
        self._rf = torch.profiler.record_function(self.name)
        self._rf.__enter__()
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)

    def end(self):
        if self._rf is not None:
            if torch.cuda.is_available():
                torch.cuda.nvtx.range_pop()
            self._rf.__exit__(None, None, None)
            self._rf = None

    __enter__ = lambda self: (self.begin(), self)[1]  # noqa: E731

    def __exit__(self, *a):
        self.end()


class _Timer:
    def __init__(self):
        self.reset()

    def reset(self):
        self.reader, self.batch, self.samples, self.steps = 0.0, 0.0, 0, 0
        self._t_batch = self._t_reader = None

    def begin(self):
        self._t_batch = self._t_reader = time.perf_counter()

    def before_reader(self):
        self._t_reader = time.perf_counter()

    def after_reader(self):
        if self._t_reader is not None:
            self.reader += time.perf_counter() - self._t_reader

    def after_step(self, num_samples):
        now = time.perf_counter()
        if self._t_batch is not None:
            self.batch += now - self._t_batch
        self._t_batch = now
        self.steps += 1
        self.samples += num_samples or 0

    def info(self, unit):
        if self.steps == 0:
            return ""
        bc = self.batch / self.steps
        ips = (self.samples / self.batch) if (self.samples and self.batch) else (1.0 / bc if bc else 0.0)
        return (f"reader_cost: {self.reader / self.steps:.5f} s batch_cost: {bc:.5f} s ips: {ips:.3f} "
                f"{unit or 'steps'}/s")


class Profiler:
    def __init__(self, *, targets=None, scheduler=None, on_trace_ready=None, record_shapes=False, profile_memory=False,
                 timer_only=False, emit_nvtx=False, custom_device_types=None, with_flops=False):
        self.targets = targets or [ProfilerTarget.CPU] + ([ProfilerTarget.GPU] if torch.cuda.is_available() else [])
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
        self._timer = _Timer()

    def _activities(self):
        acts = [torch.profiler.ProfilerActivity.CPU]
        if ProfilerTarget.GPU in self.targets and torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        return acts

    def _open(self):
        if self.timer_only or self._prof is not None:
            return
        self._prof = torch.profiler.profile(activities=self._activities(), record_shapes=self.record_shapes,
                                            profile_memory=self.profile_memory)
        self._prof.__enter__()

    def _close(self, ret):
        if self._prof is None:
            return
        self._prof.__exit__(None, None, None)
        self._last, self._prof = self._prof, None
        if ret and self.on_trace_ready is not None:
            self.on_trace_ready(self)

    def start(self):
        self._timer.begin()
        self.current_state = self.scheduler(self.step_num)
        if self.current_state in (ProfilerState.RECORD, ProfilerState.RECORD_AND_RETURN):
            self._open()

    def stop(self):
        self._close(self.current_state in (ProfilerState.RECORD, ProfilerState.RECORD_AND_RETURN))
        self.current_state = ProfilerState.CLOSED

    def step(self, num_samples=None):
        self._timer.after_step(num_samples)
        prev = self.current_state
        self.step_num += 1
        self.current_state = self.scheduler(self.step_num)
        recording = (ProfilerState.RECORD, ProfilerState.RECORD_AND_RETURN)
        if prev in recording and (prev == ProfilerState.RECORD_AND_RETURN or self.current_state not in recording):
            self._close(True)
        if self.current_state in recording:
            self._open()

    def step_info(self, unit=None):
        s = self._timer.info(unit)
        self._timer.reset()
        self._timer.begin()
        return s

    def export(self, path="", format="json"):
        p = self._last or self._prof
        if p is not None:
            p.export_chrome_trace(path)

    def summary(self, sorted_by=SortedKeys.CPUTotal, op_detail=True, thread_sep=False, time_unit="ms", views=None):
        p = self._last or self._prof
        if p is None:
            print("no profile data")
            return ""
        key = "cuda_time_total" if sorted_by.name.startswith("GPU") else "cpu_time_total"
        table = p.key_averages().table(sort_by=key, row_limit=50)
        print(table)
        return table

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *a):
        self.stop()


def load_profiler_result(filename):
    import json
    with open(filename) as f:
        return json.load(f)
