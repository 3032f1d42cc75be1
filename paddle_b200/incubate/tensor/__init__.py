"""``paddle.incubate.tensor``: segment reductions (python/paddle/incubate/tensor/math.py) and asynchronous
host offload of tensors (python/paddle/incubate/tensor/manipulation.py)."""
import torch

from ...geometric import segment_max, segment_mean, segment_min, segment_sum  # noqa: F401
from ..._core.tensor import as_tensor

__all__ = []


class _AsyncLoad:
    """A side stream for device<->pinned-host copies; ``offload`` / ``reload`` return (tensor, task) where
    ``task.wait()`` makes the current stream wait for the copy."""

    def __init__(self):
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None


class _Task:
    def __init__(self, event):
        self._e = event

    def cuda_wait(self):
        if self._e is not None:
            torch.cuda.current_stream().wait_event(self._e)

    def cpu_wait(self):
        if self._e is not None:
            self._e.synchronize()

    wait = cuda_wait


def create_async_load():
    return _AsyncLoad()


def _copy(src, dst, loader):
    if loader.stream is None:
        dst.copy_(src)
        return _Task(None)
    loader.stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(loader.stream):
        dst.copy_(src, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
    return _Task(ev)


def async_offload(src_tensor, async_load):
    s = src_tensor.as_subclass(torch.Tensor)
    dst = torch.empty(s.shape, dtype=s.dtype, device="cpu", pin_memory=torch.cuda.is_available())
    return as_tensor(dst), _copy(s, dst, async_load)


def async_reload(src_tensor, async_load):
    s = src_tensor.as_subclass(torch.Tensor)
    dst = torch.empty(s.shape, dtype=s.dtype, device="cuda" if torch.cuda.is_available() else "cpu")
    return as_tensor(dst), _copy(s, dst, async_load)


def async_offload_with_offset(src_tensor, dst_tensor, src_offset, dst_offset, offload_size, async_load):
    s = src_tensor.as_subclass(torch.Tensor).reshape(-1)[src_offset:src_offset + offload_size]
    d = dst_tensor.as_subclass(torch.Tensor).reshape(-1)[dst_offset:dst_offset + offload_size]
    return _copy(s, d, async_load)


def _npu_identity(x, format=-1):
    return x
