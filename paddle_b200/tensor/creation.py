"""Tensor creation API (python/paddle/tensor/creation.py in the reference)."""
from __future__ import annotations

import numpy as np
import torch

from .._core import dtype as _dt
from .._core.tensor import Tensor, as_tensor, to_tensor  # noqa: F401


def _shape(shape):
    if isinstance(shape, torch.Tensor):
        return tuple(int(v) for v in shape.tolist())
    if isinstance(shape, (int, np.integer)):
        return (int(shape),)
    return tuple(int(s.item()) if isinstance(s, torch.Tensor) else int(s) for s in shape)


def _mk(fn, shape, dtype, **kw):
    td = _dt.to_torch(dtype) or _dt.get_default_dtype()
    return as_tensor(fn(_shape(shape), dtype=td, device=_dt.default_device(), **kw))


def zeros(shape, dtype=None, name=None):
    return _mk(torch.zeros, shape, dtype)


def ones(shape, dtype=None, name=None):
    return _mk(torch.ones, shape, dtype)


def empty(shape, dtype=None, name=None):
    return _mk(torch.empty, shape, dtype)


def full(shape, fill_value, dtype=None, name=None):
    if dtype is None:
        dtype = "bool" if isinstance(fill_value, bool) else ("int64" if isinstance(fill_value, int) else None)
    if isinstance(fill_value, torch.Tensor):
        fill_value = fill_value.item()
    td = _dt.to_torch(dtype) or _dt.get_default_dtype()
    return as_tensor(torch.full(_shape(shape), fill_value, dtype=td, device=_dt.default_device()))


def zeros_like(x, dtype=None, name=None):
    return as_tensor(torch.zeros_like(x, dtype=_dt.to_torch(dtype)))


def ones_like(x, dtype=None, name=None):
    return as_tensor(torch.ones_like(x, dtype=_dt.to_torch(dtype)))


def empty_like(x, dtype=None, name=None):
    return as_tensor(torch.empty_like(x, dtype=_dt.to_torch(dtype)))


def full_like(x, fill_value, dtype=None, name=None):
    return as_tensor(torch.full_like(x, fill_value, dtype=_dt.to_torch(dtype)))


def arange(start=0, end=None, step=1, dtype=None, name=None):
    if end is None:
        start, end = 0, start
    vals = [v.item() if isinstance(v, torch.Tensor) else v for v in (start, end, step)]
    if dtype is None:
        dtype = "int64" if all(isinstance(v, (int, np.integer)) for v in vals) else _dt.get_default_dtype()
    return as_tensor(torch.arange(*vals, dtype=_dt.to_torch(dtype), device=_dt.default_device()))


def linspace(start, stop, num, dtype=None, name=None):
    return as_tensor(torch.linspace(float(start), float(stop), int(num), dtype=_dt.to_torch(dtype) or _dt.get_default_dtype(),
                                    device=_dt.default_device()))


def logspace(start, stop, num, base=10.0, dtype=None, name=None):
    return as_tensor(torch.logspace(float(start), float(stop), int(num), base=base,
                                    dtype=_dt.to_torch(dtype) or _dt.get_default_dtype(), device=_dt.default_device()))


def eye(num_rows, num_columns=None, dtype=None, name=None):
    return as_tensor(torch.eye(num_rows, num_columns or num_rows, dtype=_dt.to_torch(dtype) or _dt.get_default_dtype(),
                               device=_dt.default_device()))


def diag(x, offset=0, padding_value=0, name=None):
    r = torch.diag(x, offset)
    if padding_value != 0 and x.dim() == 1:
        mask = torch.diag(torch.ones_like(x, dtype=torch.bool), offset)
        r = torch.where(mask, r, torch.full_like(r, padding_value))
    return r


def diagflat(x, offset=0, name=None):
    return torch.diagflat(x, offset)


def tril(x, diagonal=0, name=None):
    return torch.tril(x, diagonal)


def triu(x, diagonal=0, name=None):
    return torch.triu(x, diagonal)


def meshgrid(*args, **kw):
    if len(args) == 1 and isinstance(args[0], (list, tuple)):
        args = tuple(args[0])
    return list(torch.meshgrid(*args, indexing="ij"))


def assign(x, output=None):
    src = x if isinstance(x, torch.Tensor) else to_tensor(x)
    if output is None:
        return src.clone()
    with torch.no_grad():
        output.copy_(src)
    return output


def clone(x, name=None):
    return x.clone()


def tril_indices(row, col, offset=0, dtype="int64"):
    return as_tensor(torch.tril_indices(row, col, offset, device=_dt.default_device()).to(_dt.to_torch(dtype)))


def triu_indices(row, col=None, offset=0, dtype="int64"):
    return as_tensor(torch.triu_indices(row, col or row, offset, device=_dt.default_device()).to(_dt.to_torch(dtype)))


def complex(real, imag, name=None):
    return torch.complex(real, imag)


def polar(abs, angle, name=None):
    return torch.polar(abs, angle)
