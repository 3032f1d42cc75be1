"""``paddle.profiler`` (python/paddle/profiler/): ``Profiler`` with scheduler states CLOSED / READY / RECORD /
RECORD_AND_RETURN driven by ``step()``, chrome-trace export, typed ``RecordEvent`` ranges (also NVTX), statistic tables
per view (overview, model phases, communication / computation overlap, operators with their kernels, kernels, memory
operations, user ranges, memory), and the reader-cost / batch-cost / ips benchmark timer.  Device and host activity
comes from the CUPTI-based activity tracer of torch."""
from . import profiler_statistic, statistic_helper, timer, utils  # noqa: F401
from .profiler import (Profiler, ProfilerResult, ProfilerState, ProfilerTarget, export_chrome_tracing, export_protobuf, get_profiler,
                       make_scheduler)
from .profiler_statistic import SortedKeys, SummaryView, TracerEventType
from .timer import benchmark
from .utils import (RecordEvent, in_profiler_mode, job_schedule_profiler_range, load_profiler_result, switch_job_schedule_profiler,
                    wrap_optimizers)

__all__ = ["ProfilerState", "ProfilerTarget", "make_scheduler", "export_chrome_tracing", "export_protobuf", "Profiler", "RecordEvent",
           "load_profiler_result", "SortedKeys", "SummaryView"]
