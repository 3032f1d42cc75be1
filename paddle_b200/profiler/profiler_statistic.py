"""Statistics over a recorded profile (python/paddle/profiler/profiler_statistic.py:40-1900): events are classified
(operator, forward / backward / optimizer phase, data loader, communication, kernel, memory copy, user range ...),
host events form a tree by containment per thread, device events hang under the host event that launched them, and
tables are built per view: overview, model (phases per step), distributed (communication / computation / overlap on
the device timeline), operator, kernel, memory manipulation, user-defined ranges and memory.

The statistics work on plain ``HostEvent`` / ``DeviceEvent`` records, so a profile can come from the activity tracer
(``events_from_torch``), from a saved chrome trace (``events_from_chrome_trace``) or be written by hand."""
from __future__ import annotations

import collections
import enum
import re
from dataclasses import dataclass, field

from .statistic_helper import intersection_ranges, merge_self_ranges, subtract_ranges, sum_ranges


class TracerEventType(enum.Enum):
    Operator = 0
    Dataloader = 1
    ProfileStep = 2
    CudaRuntime = 3
    Kernel = 4
    Memcpy = 5
    Memset = 6
    UserDefined = 7
    OperatorInner = 8
    Forward = 9
    Backward = 10
    Optimization = 11
    Communication = 12
    PythonOp = 13
    PythonUserDefined = 14


class SortedKeys(enum.Enum):
    CPUTotal = 0
    CPUAvg = 1
    CPUMax = 2
    CPUMin = 3
    GPUTotal = 4
    GPUAvg = 5
    GPUMax = 6
    GPUMin = 7


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


@dataclass
class DeviceEvent:
    name: str
    type: TracerEventType
    start_ns: int
    end_ns: int
    stream: int = 0
    device: int = 0

    @property
    def duration(self):
        return self.end_ns - self.start_ns


@dataclass
class HostEvent:
    name: str
    type: TracerEventType
    start_ns: int
    end_ns: int
    tid: int = 0
    device: list = field(default_factory=list)          # DeviceEvents launched directly by this event
    children: list = field(default_factory=list)
    input_shapes: object = None

    @property
    def duration(self):
        return self.end_ns - self.start_ns

    def all_device(self):
        out = list(self.device)
        for c in self.children:
            out += c.all_device()
        return out

    def self_time(self):
        return self.duration - sum(c.duration for c in self.children)


@dataclass
class MemEvent:
    time_ns: int
    place: str
    increase_bytes: int
    current_allocated: int = 0
    current_reserved: int = 0


# ----------------------------------------------------------------------------------------------------- classification
_COMM_PAT = re.compile(r"nccl|c10d::|all_?reduce|all_?gather|reduce_?scatter|all_?to_?all|broadcast|ag_gemm|gemm_rs|gemm_ar|"
                       r"symm_|rs_adamw|moe_dispatch|moe_combine|send|recv", re.I)
_USER_TYPES = {}                                             # range name -> type, filled by RecordEvent


def register_user_range(name, event_type):
    _USER_TYPES[name] = event_type


def classify_host(name):
    if name in _USER_TYPES:
        return _USER_TYPES[name]
    if name.startswith("ProfileStep#"):
        return TracerEventType.ProfileStep
    low = name.lower()
    if low.startswith("dataloader") or "dataloader" in low and "next" in low:
        return TracerEventType.Dataloader
    if low.startswith("cuda") or low.startswith("cu") and "launch" in low:
        return TracerEventType.CudaRuntime
    if low.startswith("optimizer.step") or low.startswith("optimizer.zero_grad"):
        return TracerEventType.Optimization
    if "evaluate_function" in low or low.endswith("backward") or low.endswith("backward0") or "backward" in low and "autograd" in low:
        return TracerEventType.Backward
    if low.startswith("nn.module:") or low.endswith(".forward"):
        return TracerEventType.Forward
    if _COMM_PAT.search(name) and ("c10d" in low or "nccl" in low or low.startswith("record_param_comms")):
        return TracerEventType.Communication
    if low.startswith("aten::") or low.startswith("pd::") or "::" in name:
        return TracerEventType.Operator
    return TracerEventType.UserDefined


def classify_device(name):
    low = name.lower()
    if low.startswith("memcpy"):
        return TracerEventType.Memcpy
    if low.startswith("memset"):
        return TracerEventType.Memset
    return TracerEventType.Kernel


def is_communication_kernel(name):
    return bool(_COMM_PAT.search(name))


# -------------------------------------------------------------------------------------------------------- event sources
def build_tree(host_events):
    """Nest host events by containment within each thread; returns the roots per thread id."""
    roots = collections.defaultdict(list)
    by_tid = collections.defaultdict(list)
    for e in host_events:
        e.children = []
        by_tid[e.tid].append(e)
    for tid, evs in by_tid.items():
        evs.sort(key=lambda e: (e.start_ns, -e.end_ns))
        stack = []
        for e in evs:
            while stack and not (stack[-1].start_ns <= e.start_ns and e.end_ns <= stack[-1].end_ns):
                stack.pop()
            (stack[-1].children if stack else roots[tid]).append(e)
            stack.append(e)
    return dict(roots)


def chrome_trace_of(prof):
    """The chrome-trace dict of a finished ``torch.profiler.profile`` (the tracer lets a window be saved once only, so
    callers keep the dict)."""
    import json
    import os
    import tempfile
    fd, path = tempfile.mkstemp(suffix=".json")
    os.close(fd)
    try:
        prof.export_chrome_trace(path)
        with open(path) as f:
            return json.load(f)
    finally:
        os.unlink(path)


def events_from_torch(prof):
    """(host events, memory events) of a finished ``torch.profiler.profile``.  The activity tracer's Python objects
    carry no start time for kernels, so the profile is written out as a chrome trace and read back."""
    return events_from_chrome_trace(chrome_trace_of(prof))


_DEVICE_CATS = {"kernel": TracerEventType.Kernel, "gpu_memcpy": TracerEventType.Memcpy, "memcpy": TracerEventType.Memcpy,
                "gpu_memset": TracerEventType.Memset, "memset": TracerEventType.Memset}


def events_from_chrome_trace(doc):
    """(host events, memory events) from a chrome-trace dict.  Complete events (``ph == "X"``) whose category names a
    kernel or a memory operation become device events and are attached to the host event that launched them:
    the one with the same ``args["correlation"]`` (the runtime call, itself nested in the operator by time), else
    the innermost host event open when the device event started, else the last host event that began before it.
    ``[memory]`` instants become memory events."""
    host, device, mem = [], [], []
    launches = {}
    for ev in doc.get("traceEvents", []):
        args = ev.get("args") or {}
        if ev.get("ph") == "i" and ev.get("name") == "[memory]":
            place = "gpu" if int(args.get("Device Type", 0) or 0) == 1 else "cpu"
            mem.append(MemEvent(int(float(ev["ts"]) * 1000), place, int(args.get("Bytes", 0) or 0), int(args.get("Total Allocated", 0) or 0),
                                int(args.get("Total Reserved", 0) or 0)))
            continue
        if ev.get("ph") != "X":
            continue
        cat = str(ev.get("cat", "")).lower()
        start = int(float(ev["ts"]) * 1000)
        end = start + int(float(ev.get("dur", 0)) * 1000)
        if cat in _DEVICE_CATS:
            d = DeviceEvent(ev["name"], _DEVICE_CATS[cat], start, end, int(args.get("stream", 0) or 0), int(args.get("device", 0) or 0))
            device.append((d, args.get("correlation")))
            continue
        if cat in ("python_function", "trace", "ac2g", "fwdbwd", "gpu_user_annotation", "overhead"):
            continue
        typ = TracerEventType.CudaRuntime if cat in ("cuda_runtime", "cuda_driver") else classify_host(ev["name"])
        h = HostEvent(ev["name"], typ, start, end, ev.get("tid", 0), input_shapes=args.get("Input Dims"))
        host.append(h)
        if "correlation" in args and typ == TracerEventType.CudaRuntime:
            launches[args["correlation"]] = h
    host.sort(key=lambda e: e.start_ns)
    for d, corr in device:
        owner = launches.get(corr) if corr is not None else None
        if owner is None:
            before = None
            for h in host:
                if h.start_ns > d.start_ns:
                    break
                if h.type == TracerEventType.ProfileStep:
                    continue
                before = h
                if d.start_ns <= h.end_ns:
                    owner = h                                  # later starts are more deeply nested
            owner = owner or before
        if owner is None:
            owner = HostEvent("[device]", TracerEventType.UserDefined, d.start_ns, d.end_ns, -1)
            host.append(owner)
        owner.device.append(d)
    return host, mem


# -------------------------------------------------------------------------------------------------------------- summaries
class TimeRangeSummary:
    """Busy time per event category on the host and on the device (ranges merged, so nested or concurrent events
    are not counted twice) plus call counts."""

    def __init__(self, host_events, step_range=None):
        self.cpu_ranges = collections.defaultdict(list)
        self.gpu_ranges = collections.defaultdict(list)
        self.calls = collections.Counter()
        for e in host_events:
            self.cpu_ranges[e.type].append((e.start_ns, e.end_ns))
            self.calls[e.type] += 1
            for d in e.device:
                self.gpu_ranges[d.type].append((d.start_ns, d.end_ns))
                self.calls[d.type] += 1
                if is_communication_kernel(d.name):
                    self.gpu_ranges[TracerEventType.Communication].append((d.start_ns, d.end_ns))
        self.cpu_times = {t: sum_ranges(merge_self_ranges(r)) for t, r in self.cpu_ranges.items()}
        self.gpu_times = {t: sum_ranges(merge_self_ranges(r)) for t, r in self.gpu_ranges.items()}
        lo = min((e.start_ns for e in host_events), default=0)
        hi = max([e.end_ns for e in host_events] + [d.end_ns for e in host_events for d in e.device], default=0)
        self.total_ns = (step_range[1] - step_range[0]) if step_range else hi - lo

    def get_cpu_range_sum(self, t):
        return self.cpu_times.get(t, 0)

    def get_gpu_range_sum(self, t):
        return self.gpu_times.get(t, 0)


class DistributedSummary:
    """Device timeline split into communication and computation kernels: how long each kept the GPU busy and how
    much of the communication ran under computation (the overlap a fused or side-stream collective is meant to buy)."""

    def __init__(self, host_events):
        comm, comp = [], []
        for e in host_events:
            for d in e.device:
                if d.type != TracerEventType.Kernel:
                    continue
                (comm if is_communication_kernel(d.name) else comp).append((d.start_ns, d.end_ns))
        self.communication_range = merge_self_ranges(comm)
        self.computation_range = merge_self_ranges(comp)
        self.overlap_range = intersection_ranges(self.communication_range, self.computation_range, True)
        self.exposed_communication_range = subtract_ranges(self.communication_range, self.computation_range, True)
        self.communication_ns = sum_ranges(self.communication_range)
        self.computation_ns = sum_ranges(self.computation_range)
        self.overlap_ns = sum_ranges(self.overlap_range)
        self.exposed_ns = sum_ranges(self.exposed_communication_range)


@dataclass
class _Item:
    name: str
    call: int = 0
    cpu_time: int = 0
    max_cpu_time: int = 0
    min_cpu_time: int = 1 << 62
    gpu_time: int = 0
    max_gpu_time: int = 0
    min_gpu_time: int = 1 << 62
    devices: dict = field(default_factory=dict)           # kernel name -> _Item (operator detail)

    def add(self, cpu, gpu):
        self.call += 1
        self.cpu_time += cpu
        self.max_cpu_time, self.min_cpu_time = max(self.max_cpu_time, cpu), min(self.min_cpu_time, cpu)
        self.gpu_time += gpu
        self.max_gpu_time, self.min_gpu_time = max(self.max_gpu_time, gpu), min(self.min_gpu_time, gpu)

    avg_cpu_time = property(lambda s: s.cpu_time / s.call if s.call else 0)
    avg_gpu_time = property(lambda s: s.gpu_time / s.call if s.call else 0)


class EventSummary:
    """Per-name statistics: operators (with the kernels each launched), kernels, memory copies / sets, user ranges,
    and the model phases (data loader, forward, backward, optimizer, other) per profiled step."""

    def __init__(self, host_events):
        self.items = {}                   # operators
        self.kernel_items = {}
        self.memory_manipulation_items = {}
        self.userdefined_items = {}
        self.model_perspective_items = {}
        roots = build_tree(host_events)
        for tid, rs in roots.items():
            for r in rs:
                self._walk(r, inside_op=False)
        for e in host_events:
            for d in e.device:
                table = self.kernel_items if d.type == TracerEventType.Kernel else self.memory_manipulation_items
                table.setdefault(d.name, _Item(d.name)).add(0, d.duration)
        self._model_view(host_events)

    def _walk(self, e, inside_op):
        if e.type in (TracerEventType.Operator, TracerEventType.Communication) and not inside_op:
            it = self.items.setdefault(e.name, _Item(e.name))
            devs = e.all_device()
            it.add(e.duration, sum(d.duration for d in devs))
            for d in devs:
                it.devices.setdefault(d.name, _Item(d.name)).add(0, d.duration)
            inside_op = True
        elif e.type in (TracerEventType.UserDefined, TracerEventType.PythonUserDefined):
            self.userdefined_items.setdefault(e.name, _Item(e.name)).add(e.duration, sum(d.duration for d in e.all_device()))
        for c in e.children:
            self._walk(c, inside_op)

    def _model_view(self, host_events):
        phases = {TracerEventType.Dataloader: "Dataloader", TracerEventType.Forward: "Forward", TracerEventType.Backward: "Backward",
                  TracerEventType.Optimization: "Optimization"}
        steps = [e for e in host_events if e.type == TracerEventType.ProfileStep]
        total = self.model_perspective_items.setdefault("ProfileStep", _Item("ProfileStep"))
        covered_cpu, covered_gpu = 0, 0
        roots = build_tree(host_events)

        def outermost(e, out):
            if e.type in phases:
                out.append(e)
                return
            for c in e.children:
                outermost(c, out)
        tops = []
        for rs in roots.values():
            for r in rs:
                outermost(r, tops)
        for e in tops:
            gpu = sum(d.duration for d in e.all_device())
            self.model_perspective_items.setdefault(phases[e.type], _Item(phases[e.type])).add(e.duration, gpu)
            covered_cpu += e.duration
            covered_gpu += gpu
        all_gpu = sum(d.duration for e in host_events for d in e.device)
        if steps:
            for s in steps:
                total.add(s.duration, 0)
            total.gpu_time = all_gpu
        else:
            lo = min((e.start_ns for e in host_events), default=0)
            hi = max((e.end_ns for e in host_events), default=0)
            total.add(hi - lo, all_gpu)
        other = self.model_perspective_items.setdefault("Others", _Item("Others"))
        other.add(max(total.cpu_time - covered_cpu, 0), max(all_gpu - covered_gpu, 0))


class MemorySummary:
    """Peak allocated bytes per place, and the largest single increases."""

    def __init__(self, mem_events):
        self.peak_allocated = collections.defaultdict(int)
        self.allocated = collections.defaultdict(int)
        self.alloc_calls = collections.Counter()
        self.free_calls = collections.Counter()
        for m in sorted(mem_events, key=lambda m: m.time_ns):
            self.allocated[m.place] += m.increase_bytes
            self.peak_allocated[m.place] = max(self.peak_allocated[m.place], self.allocated[m.place], m.current_allocated)
            (self.alloc_calls if m.increase_bytes > 0 else self.free_calls)[m.place] += 1


class StatisticData:
    def __init__(self, host_events, mem_events=()):
        self.host_events = list(host_events)
        self.time_range_summary = TimeRangeSummary(self.host_events)
        self.event_summary = EventSummary(self.host_events)
        self.distributed_summary = DistributedSummary(self.host_events)
        self.memory_summary = MemorySummary(mem_events)


# ------------------------------------------------------------------------------------------------------------------ tables
def _format_time(ns, unit="ms", precision=2):
    div = {"s": 1e9, "ms": 1e6, "us": 1e3, "ns": 1.0}[unit]
    return f"{ns / div:.{precision}f}"


def _format_large_number(n, precision=2):
    for lim, suffix in ((1e12, "T"), (1e9, "G"), (1e6, "M"), (1e3, "K")):
        if abs(n) >= lim:
            return f"{n / lim:.{precision}f}{suffix}"
    return f"{n:.0f}"


def _table(title, header, rows):
    if not rows:
        return ""
    widths = [max(len(str(h)), *(len(str(r[i])) for r in rows)) for i, h in enumerate(header)]
    widths = [min(w, 75) for w in widths]
    line = "-" * (sum(widths) + 2 * len(widths))
    fmt = lambda cells: "  ".join(str(c)[:w].ljust(w) if i == 0 else str(c)[:w].rjust(w) for i, (c, w) in enumerate(zip(cells, widths)))
    out = [line, title.center(len(line)), line, fmt(header), line]
    out += [fmt(r) for r in rows]
    out.append(line)
    return "\n".join(out) + "\n"


_SORT = {SortedKeys.CPUTotal: lambda i: i.cpu_time, SortedKeys.CPUAvg: lambda i: i.avg_cpu_time, SortedKeys.CPUMax: lambda i: i.max_cpu_time,
         SortedKeys.CPUMin: lambda i: i.min_cpu_time, SortedKeys.GPUTotal: lambda i: i.gpu_time, SortedKeys.GPUAvg: lambda i: i.avg_gpu_time,
         SortedKeys.GPUMax: lambda i: i.max_gpu_time, SortedKeys.GPUMin: lambda i: i.min_gpu_time}


def _item_rows(items, sorted_by, unit, total_cpu, total_gpu, detail=False, row_limit=100):
    rows = []
    for it in sorted(items.values(), key=_SORT[sorted_by], reverse=True)[:row_limit]:
        t = lambda v: _format_time(v, unit)
        rows.append([it.name, it.call, f"{t(it.cpu_time)} / {t(it.avg_cpu_time)} / {t(it.max_cpu_time)} / {t(it.min_cpu_time if it.call else 0)}",
                     f"{100 * it.cpu_time / total_cpu:.2f}" if total_cpu else "-",
                     f"{t(it.gpu_time)} / {t(it.avg_gpu_time)} / {t(it.max_gpu_time)} / {t(it.min_gpu_time if it.call else 0)}",
                     f"{100 * it.gpu_time / total_gpu:.2f}" if total_gpu else "-"])
        if detail:
            for k in sorted(it.devices.values(), key=lambda i: i.gpu_time, reverse=True):
                rows.append(["    " + k.name, k.call, "-", "-",
                             f"{t(k.gpu_time)} / {t(k.avg_gpu_time)} / {t(k.max_gpu_time)} / {t(k.min_gpu_time)}",
                             f"{100 * k.gpu_time / total_gpu:.2f}" if total_gpu else "-"])
    return rows


def _build_table(statistic_data, sorted_by=SortedKeys.CPUTotal, op_detail=True, thread_sep=False, time_unit="ms", row_limit=100,
                 max_src_column_width=75, views=None):
    """The report as text; ``views`` (one ``SummaryView`` or a list) restricts it."""
    if views is not None and not isinstance(views, (list, tuple)):
        views = [views]
    want = lambda v: views is None or v in views
    sd, out = statistic_data, []
    trs, es = sd.time_range_summary, sd.event_summary
    total = trs.total_ns or 1
    t = lambda v: _format_time(v, time_unit)
    hdr4 = ["Name", "Calls", f"CPU Total / Avg / Max / Min ({time_unit})", "Ratio (%)", f"GPU Total / Avg / Max / Min ({time_unit})", "Ratio (%)"]
    if want(SummaryView.OverView):
        rows = []
        for typ in TracerEventType:
            c, g = trs.get_cpu_range_sum(typ), trs.get_gpu_range_sum(typ)
            if c or g:
                rows.append([typ.name, trs.calls.get(typ, 0), t(c), f"{100 * c / total:.2f}", t(g), f"{100 * g / total:.2f}"])
        out.append(_table("Overview Summary", ["Event Type", "Calls", f"CPU Time ({time_unit})", "Ratio (%)", f"GPU Time ({time_unit})", "Ratio (%)"], rows))
    if want(SummaryView.ModelView):
        items = es.model_perspective_items
        tot = items.get("ProfileStep")
        rows = []
        for name in ("ProfileStep", "Dataloader", "Forward", "Backward", "Optimization", "Others"):
            it = items.get(name)
            if it is None or not it.call:
                continue
            rows.append([name, it.call, t(it.cpu_time), f"{100 * it.cpu_time / tot.cpu_time:.2f}" if tot and tot.cpu_time else "-",
                         t(it.gpu_time), f"{100 * it.gpu_time / tot.gpu_time:.2f}" if tot and tot.gpu_time else "-"])
        out.append(_table("Model Summary", ["Name", "Calls", f"CPU Total ({time_unit})", "Ratio (%)", f"GPU Total ({time_unit})", "Ratio (%)"], rows))
    if want(SummaryView.DistributedView):
        ds = sd.distributed_summary
        if ds.communication_ns:
            rows = [["ProfileStep", t(total), "100.00"],
                    ["  Communication", t(ds.communication_ns), f"{100 * ds.communication_ns / total:.2f}"],
                    ["  Computation", t(ds.computation_ns), f"{100 * ds.computation_ns / total:.2f}"],
                    ["  Overlap", t(ds.overlap_ns), f"{100 * ds.overlap_ns / total:.2f}"],
                    ["  Exposed communication", t(ds.exposed_ns), f"{100 * ds.exposed_ns / total:.2f}"]]
            out.append(_table("Distribution Summary", ["Name", f"Total Time ({time_unit})", "Ratio (%)"], rows))
    total_cpu = sum(i.cpu_time for i in es.items.values())
    total_gpu = sum(i.gpu_time for i in es.kernel_items.values()) + sum(i.gpu_time for i in es.memory_manipulation_items.values())
    if want(SummaryView.OperatorView):
        out.append(_table("Operator Summary", hdr4, _item_rows(es.items, sorted_by, time_unit, total_cpu, total_gpu, op_detail, row_limit)))
    if want(SummaryView.KernelView):
        key = sorted_by if sorted_by.name.startswith("GPU") else SortedKeys.GPUTotal
        rows = [[r[0], r[1], r[4], r[5]] for r in _item_rows(es.kernel_items, key, time_unit, 0, total_gpu, False, row_limit)]
        out.append(_table("Kernel Summary", ["Name", "Calls", f"GPU Total / Avg / Max / Min ({time_unit})", "Ratio (%)"], rows))
    if want(SummaryView.MemoryManipulationView):
        rows = [[r[0], r[1], r[4], r[5]] for r in _item_rows(es.memory_manipulation_items, SortedKeys.GPUTotal, time_unit, 0, total_gpu, False, row_limit)]
        out.append(_table("Memory Manipulation Summary", ["Name", "Calls", f"GPU Total / Avg / Max / Min ({time_unit})", "Ratio (%)"], rows))
    if want(SummaryView.UDFView):
        ucpu = sum(i.cpu_time for i in es.userdefined_items.values())
        out.append(_table("UserDefined Summary", hdr4, _item_rows(es.userdefined_items, sorted_by, time_unit, ucpu, total_gpu, False, row_limit)))
    if want(SummaryView.MemoryView):
        ms = sd.memory_summary
        rows = [[place, ms.alloc_calls[place], ms.free_calls[place], _format_large_number(ms.peak_allocated[place])]
                for place in sorted(ms.peak_allocated)]
        out.append(_table("Memory Summary", ["Place", "Allocations", "Frees", "Peak Allocated (bytes)"], rows))
    return "\n".join(s for s in out if s)
