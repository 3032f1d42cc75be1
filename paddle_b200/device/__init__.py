"""``paddle.device``: device selection, streams / events, memory statistics, CUDA graphs
(python/paddle/device/__init__.py, device/cuda/__init__.py, device/cuda/graphs.py) mapped on torch.cuda."""
from __future__ import annotations

import torch

from .._core.dtype import get_device, set_device  # noqa: F401
from . import cuda  # noqa: F401

Stream = torch.cuda.Stream
Event = torch.cuda.Event


def get_all_device_type():
    return ["cpu"] + (["gpu"] if torch.cuda.is_available() else [])


def get_available_device():
    return ["cpu"] + [f"gpu:{i}" for i in range(torch.cuda.device_count())]


def get_all_custom_device_type():
    return []


def get_available_custom_device():
    return []


def is_compiled_with_cuda():
    return True


def is_compiled_with_rocm():
    return False


def is_compiled_with_xpu():
    return False


def is_compiled_with_custom_device(name=None):
    return False


def is_compiled_with_cinn():
    return False


def synchronize(device=None):
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def current_stream(device=None):
    return torch.cuda.current_stream()


def set_stream(stream):
    prev = torch.cuda.current_stream()
    torch.cuda.set_stream(stream)
    return prev


def stream_guard(stream):
    return torch.cuda.stream(stream)


def get_cudnn_version():
    v = torch.backends.cudnn.version() if torch.backends.cudnn.is_available() else None
    return v


class XPUPlace:
    def __init__(self, dev_id=0):
        raise RuntimeError("XPU devices are not supported")


class IPUPlace:
    def __init__(self):
        raise RuntimeError("IPU devices are not supported")


def is_compiled_with_ipu():
    return False


def is_compiled_with_distribute():
    return torch.distributed.is_available()
