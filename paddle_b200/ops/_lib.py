"""ctypes loader for the native libraries plus the device-side status word.

The kernels are exported with a C ABI (``pd_*`` symbols).  Python passes raw device pointers, sizes
and the current CUDA stream.  On a machine with a GPU a missing library is a hard error: the ops in
this package never fall back silently to another implementation.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_LIB_DIR = os.path.join(_PKG, "lib")
_lock = threading.Lock()
_kernels = None
_runtime = None


class NativeLibraryError(RuntimeError):
    pass


def _timeout_base():
    from ..framework.errors import ExecutionTimeoutError
    return ExecutionTimeoutError


class KernelStatusError(_timeout_base()):
    """A kernel gave up on a bounded wait (or rejected its arguments) and wrote a status word.  An
    ``ExecutionTimeoutError`` (error code 8), hence a ``RuntimeError``."""


def _load(name: str, builder: str):
    path = os.path.join(_LIB_DIR, name)
    if not os.path.exists(path):
        try:
            from . import build as _build
            getattr(_build, builder)()
        except Exception as e:  # noqa: BLE001
            raise NativeLibraryError(
                f"{name} is not built and building it failed: {e}. "
                f"Run `python -m paddle_b200.ops.build`.") from e
    try:
        return ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    except OSError as e:
        raise NativeLibraryError(f"cannot load {path}: {e}") from e


def kernels() -> ctypes.CDLL:
    """The CUDA kernel library (``libpd_kernels.so``)."""
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                if os.environ.get("PD_DEBUG_BOUNDS") == "1":
                    # checked build: every TMA / bulk copy is validated before it is issued (sm100_prims.cuh)
                    path = os.path.join(_LIB_DIR, "libpd_kernels_dbg.so")
                    if not os.path.exists(path):
                        from . import build as _build
                        _build.build_kernels(debug_bounds=True)
                    _kernels = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
                else:
                    _kernels = _load("libpd_kernels.so", "build_kernels")
    return _kernels


def debug_bounds_violation():
    """First violation recorded by the ``PD_DEBUG_BOUNDS=1`` build since the last call, as a dict, or None."""
    k = kernels()
    if not hasattr(k, "pd_debug_bounds_read"):
        raise RuntimeError("the loaded kernel library is not the debug-bounds build (set PD_DEBUG_BOUNDS=1)")
    rec = (ctypes.c_int * 8)()
    check(k.pd_debug_bounds_read(rec), "pd_debug_bounds_read")
    if rec[0] == 0:
        return None
    kinds = {1: "tma_load_2d", 2: "tma_load_3d", 3: "tma_load_4d", 11: "tma_store_2d", 12: "tma_store_3d",
             13: "tma_store_4d", 21: "tma_reduce_add_2d", 23: "tma_reduce_add_4d", 31: "bulk_load", 32: "bulk_store"}
    return {"copy": kinds.get(rec[0], rec[0]), "x": rec[1], "y": rec[2], "block": rec[3], "thread": rec[4]}


def runtime() -> ctypes.CDLL:
    """The host runtime library (``libpd_runtime.so``)."""
    global _runtime
    if _runtime is None:
        with _lock:
            if _runtime is None:
                san = os.environ.get("PD_RUNTIME_SANITIZER")
                if san:
                    from . import build as _build
                    _build.build_runtime(sanitize=san)
                    _runtime = _load(f"libpd_runtime_{san}.so", "build_runtime")
                else:
                    _runtime = _load("libpd_runtime.so", "build_runtime")
                _runtime.pd_flag_set.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
                _runtime.pd_flag_set.restype = None
                from ..framework import flags as _flags
                _flags.sync_native()
    return _runtime


def have_gpu() -> bool:
    return torch.cuda.is_available()


# ---------------------------------------------------------------------------------------- helpers
c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float


def ptr(t) -> ctypes.c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def stream() -> ctypes.c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_LAUNCH_ERRORS = {
    -1: "bad shape", -2: "pointer/stride alignment", -3: "TMA tensor-map encoding failed",
    -4: "CUDA launch error", -5: "size beyond the supported maximum",
}


def check(rc: int, what: str):
    """Turn a launcher return code into a typed error (``framework/errors.py``): bad shape / alignment ->
    InvalidArgumentError (a ValueError), beyond the supported size -> OutOfRangeError, tensor-map or CUDA launch failure
    -> ExternalError; all of them are RuntimeErrors as well."""
    if rc != 0:
        from ..framework import errors
        cls = errors.LAUNCH_ERROR_CLASSES.get(rc, errors.LaunchExternal)
        raise cls(f"{what}: native launcher returned {rc} ({_LAUNCH_ERRORS.get(rc, 'unknown')})")
    if _sync_launches[0]:
        # FLAGS_benchmark / FLAGS_check_kernel_launch: wait for the kernel and surface its status word at the call site
        if torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
            torch.cuda.synchronize()
            check_status()


# switched by framework.flags when FLAGS_benchmark or FLAGS_check_kernel_launch changes
_sync_launches = [False]


# One 4-int status word per device: {code, block, site, detail}; written by kernels whose bounded
# waits expire.  Checked by `check_status()` (tests, step boundaries), never on the hot path.
_status = {}


def status_buffer(device=None) -> torch.Tensor:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index
    buf = _status.get(key)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=dev)
        _status[key] = buf
    return buf


def check_status(device=None, reset: bool = True):
    buf = status_buffer(device)
    vals = buf.tolist()  # synchronises
    if vals[0] != 0:
        if reset:
            buf.zero_()
        names = {1: "mbarrier wait timed out", 2: "flag wait timed out", 3: "bad argument"}
        raise KernelStatusError(
            f"kernel status {vals[0]} ({names.get(vals[0], '?')}): block={vals[1]} site={vals[2]} detail={vals[3]}")
