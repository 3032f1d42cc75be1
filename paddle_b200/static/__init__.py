"""``paddle.static``: the pieces of the static-graph API that dynamic-to-static capture needs:
``InputSpec`` (python/paddle/static/input.py) and save/load of captured programs."""
from __future__ import annotations

import numpy as np

from .._core import dtype as _dt


class InputSpec:
    def __init__(self, shape=None, dtype="float32", name=None, stop_gradient=False):
        self.shape = tuple(shape) if shape is not None else None
        self.dtype = _dt.to_torch(dtype)
        self.name = name
        self.stop_gradient = stop_gradient

    @classmethod
    def from_tensor(cls, tensor, name=None):
        return cls(list(tensor.shape), tensor.dtype, name or getattr(tensor, "name", None))

    @classmethod
    def from_numpy(cls, ndarray, name=None):
        return cls(ndarray.shape, ndarray.dtype, name)

    def batch(self, batch_size):
        self.shape = (batch_size, *self.shape)
        return self

    def unbatch(self):
        self.shape = self.shape[1:]
        return self

    def matches(self, tensor):
        if self.shape is None:
            return True
        if len(self.shape) != tensor.dim():
            return False
        return all(s is None or s == -1 or s == t for s, t in zip(self.shape, tensor.shape)) and tensor.dtype == self.dtype

    def __repr__(self):
        return f"InputSpec(shape={self.shape}, dtype={_dt.to_name(self.dtype)}, name={self.name})"

    def __hash__(self):
        return hash((self.shape, self.dtype, self.name))

    def __eq__(self, o):
        return isinstance(o, InputSpec) and (self.shape, self.dtype, self.name) == (o.shape, o.dtype, o.name)


def save_inference_model(path_prefix, feed_vars, fetch_vars, executor=None, **kw):
    from ..jit import save
    layer = kw.get("program") or kw.get("layer")
    if layer is None:
        raise ValueError("pass the captured layer as `layer=`")
    save(layer, path_prefix, input_spec=feed_vars)


def load_inference_model(path_prefix, executor=None, **kw):
    from ..jit import load
    return load(path_prefix)
