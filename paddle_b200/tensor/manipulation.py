"""Shape / layout manipulation API (python/paddle/tensor/manipulation.py in the reference)."""
from __future__ import annotations

import numpy as np
import torch

from .._core import dtype as _dt
from .._core.tensor import Tensor, as_tensor, to_tensor
from .creation import _shape


def cast(x, dtype):
    return x.to(_dt.to_torch(dtype))


def reshape(x, shape, name=None):
    return Tensor.reshape(as_tensor(x), list(_shape(shape)))


def reshape_(x, shape, name=None):
    return Tensor.reshape_(as_tensor(x), list(_shape(shape)))


view = reshape


def transpose(x, perm, name=None):
    return x.permute(*perm)


def moveaxis(x, source, destination, name=None):
    return torch.movedim(x, source, destination)


def swapaxes(x, axis0, axis1):
    return torch.swapaxes(x, axis0, axis1)


def t(x, name=None):
    return x if x.dim() < 2 else torch.t(x)


def concat(x, axis=0, name=None):
    if isinstance(axis, torch.Tensor):
        axis = int(axis.item())
    return torch.cat(list(x), dim=axis)


def stack(x, axis=0, name=None):
    return torch.stack(list(x), dim=axis)


def hstack(x, name=None):
    return torch.hstack(list(x))


def vstack(x, name=None):
    return torch.vstack(list(x))


def dstack(x, name=None):
    return torch.dstack(list(x))


def split(x, num_or_sections, axis=0, name=None):
    if isinstance(axis, torch.Tensor):
        axis = int(axis.item())
    return Tensor.split(as_tensor(x), num_or_sections, axis)


def tensor_split(x, num_or_indices, axis=0, name=None):
    return list(torch.tensor_split(x, num_or_indices, dim=axis))


def chunk(x, chunks, axis=0, name=None):
    return list(torch.chunk(x, chunks, dim=axis))


def unbind(input, axis=0):
    return list(torch.unbind(input, axis))


def unstack(x, axis=0, num=None):
    return list(torch.unbind(x, axis))


def squeeze(x, axis=None, name=None):
    return Tensor.squeeze(as_tensor(x), axis)


def unsqueeze(x, axis, name=None):
    if isinstance(axis, torch.Tensor):
        axis = axis.tolist()
    return Tensor.unsqueeze(as_tensor(x), axis)


def flatten(x, start_axis=0, stop_axis=-1, name=None):
    return torch.flatten(x, start_axis, stop_axis)


def unflatten(x, axis, shape, name=None):
    return torch.unflatten(x, axis, tuple(_shape(shape)))


def expand(x, shape, name=None):
    return x.expand(*_shape(shape))


def expand_as(x, y, name=None):
    return x.expand_as(y)


def broadcast_to(x, shape, name=None):
    return torch.broadcast_to(x, _shape(shape))


def broadcast_tensors(input, name=None):
    return list(torch.broadcast_tensors(*input))


def broadcast_shape(x_shape, y_shape):
    return list(torch.broadcast_shapes(tuple(x_shape), tuple(y_shape)))


def tile(x, repeat_times, name=None):
    return x.repeat(*_shape(repeat_times))


def repeat_interleave(x, repeats, axis=None, name=None):
    return torch.repeat_interleave(x, repeats, dim=axis)


def flip(x, axis, name=None):
    return torch.flip(x, [axis] if isinstance(axis, int) else list(axis))


def rot90(x, k=1, axes=(0, 1), name=None):
    return torch.rot90(x, k, list(axes))


def roll(x, shifts, axis=None, name=None):
    return torch.roll(x, shifts, axis)


def gather(x, index, axis=0, name=None):
    if isinstance(axis, torch.Tensor):
        axis = int(axis.item())
    return torch.index_select(x, axis, index.reshape(-1))


def gather_nd(x, index, name=None):
    idx = index.long()
    k = idx.shape[-1]
    return x[tuple(idx[..., i] for i in range(k))]


def take_along_axis(arr, indices, axis, broadcast=True):
    return torch.take_along_dim(arr, indices, axis)


def put_along_axis(arr, indices, values, axis, reduce="assign", include_self=True, broadcast=True):
    if not isinstance(values, torch.Tensor):
        values = torch.full_like(indices, values, dtype=arr.dtype)
    values = values.expand_as(indices) if values.shape != indices.shape else values
    if reduce == "assign":
        return torch.scatter(arr, axis, indices, values)
    red = {"add": "sum", "mul": "prod", "multiply": "prod", "mean": "mean", "amin": "amin", "amax": "amax"}[reduce]
    return torch.scatter_reduce(arr, axis, indices, values, red, include_self=include_self)


def scatter(x, index, updates, overwrite=True, name=None):
    idx = index.reshape(-1).long()
    if overwrite:
        out = x.clone()
        out[idx] = updates
        return out
    out = x.clone()
    out[idx] = 0
    return out.index_add(0, idx, updates)


def scatter_(x, index, updates, overwrite=True, name=None):
    x.copy_(scatter(x, index, updates, overwrite))
    return x


def scatter_nd_add(x, index, updates, name=None):
    idx = index.long()
    k = idx.shape[-1]
    out = x.clone()
    out.index_put_(tuple(idx[..., i] for i in range(k)), updates, accumulate=True)
    return out


def scatter_nd(index, updates, shape, name=None):
    return scatter_nd_add(torch.zeros(_shape(shape), dtype=updates.dtype, device=updates.device), index, updates)


def index_add(x, index, axis, value, name=None):
    return torch.index_add(x, axis, index, value)


def index_put(x, indices, value, accumulate=False, name=None):
    return torch.index_put(x, tuple(indices), value, accumulate)


def index_fill(x, index, axis, value, name=None):
    return torch.index_fill(x, axis, index, value)


def slice(input, axes, starts, ends):
    sl = [builtins_slice(None)] * input.dim()
    for a, s, e in zip(axes, starts, ends):
        s = int(s.item()) if isinstance(s, torch.Tensor) else s
        e = int(e.item()) if isinstance(e, torch.Tensor) else e
        sl[a] = builtins_slice(s, e)
    return input[tuple(sl)]


import builtins as _b  # noqa: E402

builtins_slice = _b.slice


def strided_slice(x, axes, starts, ends, strides, name=None):
    sl = [builtins_slice(None)] * x.dim()
    for a, s, e, st in zip(axes, starts, ends, strides):
        sl[a] = builtins_slice(s, e, st)
    return x[tuple(sl)]


def crop(x, shape=None, offsets=None, name=None):
    offsets = offsets or [0] * x.dim()
    shape = _shape(shape)
    sl = tuple(builtins_slice(o, o + (s if s != -1 else x.shape[i] - o)) for i, (o, s) in enumerate(zip(offsets, shape)))
    return x[sl]


def pad(x, pad, mode="constant", value=0.0, data_format="NCHW", name=None):
    from ..nn.functional import pad as _pad
    return _pad(x, pad, mode, value, data_format)


def shard_index(input, index_num, nshards, shard_id, ignore_value=-1):
    size = (index_num + nshards - 1) // nshards
    lo, hi = shard_id * size, (shard_id + 1) * size
    return torch.where((input >= lo) & (input < hi), input - lo, torch.full_like(input, ignore_value))


def numel(x, name=None):
    return as_tensor(torch.tensor(torch.Tensor.numel(x), dtype=torch.int64))


def shape(x):
    return as_tensor(torch.tensor(list(x.shape), dtype=torch.int32))


def rank(x):
    return as_tensor(torch.tensor(x.dim(), dtype=torch.int32))


def as_complex(x, name=None):
    return torch.view_as_complex(x)


def as_real(x, name=None):
    return torch.view_as_real(x)


def as_strided(x, shape, stride, offset=0, name=None):
    return torch.as_strided(x, tuple(shape), tuple(stride), offset)


def view_as(x, other, name=None):
    return x.view_as(other)


def atleast_1d(*inputs, name=None):
    r = torch.atleast_1d(*inputs)
    return list(r) if isinstance(r, tuple) else r


def atleast_2d(*inputs, name=None):
    r = torch.atleast_2d(*inputs)
    return list(r) if isinstance(r, tuple) else r


def atleast_3d(*inputs, name=None):
    r = torch.atleast_3d(*inputs)
    return list(r) if isinstance(r, tuple) else r


def masked_scatter(x, mask, value, name=None):
    return torch.masked_scatter(x, mask, value)


def select_scatter(x, values, axis, index, name=None):
    return torch.select_scatter(x, values, axis, index)


def diagonal_scatter(x, y, offset=0, axis1=0, axis2=1, name=None):
    return torch.diagonal_scatter(x, y, offset, axis1, axis2)


def tolist(x):
    return x.tolist()
