"""``paddle.device.cuda``"""
from __future__ import annotations

import contextlib

import torch

Stream = torch.cuda.Stream
Event = torch.cuda.Event


def device_count():
    return torch.cuda.device_count()


def current_stream(device=None):
    return torch.cuda.current_stream()


def synchronize(device=None):
    torch.cuda.synchronize()


def stream_guard(stream):
    return torch.cuda.stream(stream)


def empty_cache():
    torch.cuda.empty_cache()


def memory_allocated(device=None):
    return torch.cuda.memory_allocated()


def max_memory_allocated(device=None):
    return torch.cuda.max_memory_allocated()


def memory_reserved(device=None):
    return torch.cuda.memory_reserved()


def max_memory_reserved(device=None):
    return torch.cuda.max_memory_reserved()


def reset_max_memory_allocated(device=None):
    torch.cuda.reset_peak_memory_stats()


reset_max_memory_reserved = reset_max_memory_allocated


def get_device_properties(device=None):
    return torch.cuda.get_device_properties(torch.cuda.current_device())


def get_device_name(device=None):
    return torch.cuda.get_device_name()


def get_device_capability(device=None):
    return torch.cuda.get_device_capability()


from . import graphs, streams  # noqa: E402,F401
from .graphs import CUDAGraph, cuda_graph_capture, is_cuda_graph_supported, wrap_cuda_graph  # noqa: E402,F401
