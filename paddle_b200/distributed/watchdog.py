"""Host-side communication watchdog (reference: FLAGS_enable_async_trace,
paddle/phi/core/distributed/comm_task_manager.cc).  Collectives register a task when issued and mark it
started / finished from CUDA-event queries or work completion; a native background thread reports tasks
that exceed the timeout, saying whether they never started or started and did not finish and what the
group's last completed collective was.  It never blocks the GPU."""
from __future__ import annotations

import ctypes

from ..ops import _lib

_started = False


class CommTimeoutError(RuntimeError):
    pass


def start(timeout_s=1800.0, poll_ms=100):
    global _started
    rt = _lib.runtime()
    rt.pd_watchdog_task_create.restype = ctypes.c_int64
    rt.pd_watchdog_start(int(timeout_s * 1000), int(poll_ms))
    _started = True


def stop():
    global _started
    if _started:
        _lib.runtime().pd_watchdog_stop()
        _started = False


def enabled():
    return _started


def task_create(group_id, name, nbytes):
    return int(_lib.runtime().pd_watchdog_task_create(int(group_id), name.encode(), ctypes.c_int64(nbytes)))


def task_started(tid):
    _lib.runtime().pd_watchdog_task_started(ctypes.c_int64(tid))


def task_finished(tid):
    _lib.runtime().pd_watchdog_task_finished(ctypes.c_int64(tid))


def poll():
    """Returns the next timeout report or None."""
    buf = ctypes.create_string_buffer(1024)
    n = _lib.runtime().pd_watchdog_poll(buf, 1024)
    return buf.value.decode() if n > 0 else None


def check():
    v = poll()
    if v is not None:
        raise CommTimeoutError(v)


def inflight():
    return _lib.runtime().pd_watchdog_inflight()
