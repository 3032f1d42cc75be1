import torch.utils.dlpack as _d

from .._core.tensor import as_tensor


def to_dlpack(x):
    return _d.to_dlpack(x)


def from_dlpack(capsule):
    return as_tensor(_d.from_dlpack(capsule))
