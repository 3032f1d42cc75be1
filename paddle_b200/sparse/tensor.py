"""The tensor type of ``paddle.sparse``: a COO or CSR tensor carried by torch's sparse layouts, presented with the
reference's interface (``indices() / values() / crows() / cols() / nnz() / to_dense() / to_sparse_coo() /
to_sparse_csr()``, list ``shape``, ``stop_gradient``, the reference's print-out).  torch functions called on it
dispatch through ``__torch_function__`` to the wrapped tensor, so the operators of this package treat both alike."""
from __future__ import annotations

import torch

from .._core import dtype as _dt
from .._core.tensor import Tensor, as_tensor


def unwrap(o):
    if isinstance(o, SparseTensor):
        return o._t
    if isinstance(o, (list, tuple)):
        return type(o)(unwrap(v) for v in o)
    if isinstance(o, dict):
        return {k: unwrap(v) for k, v in o.items()}
    return o


def wrap(o):
    if isinstance(o, torch.Tensor):
        if o.layout in (torch.sparse_coo, torch.sparse_csr):
            return SparseTensor(o)
        return o if isinstance(o, Tensor) else as_tensor(o)
    if isinstance(o, tuple):
        return tuple(wrap(v) for v in o)
    if isinstance(o, list):
        return [wrap(v) for v in o]
    if isinstance(o, torch.Size):
        return list(o)
    return o


def api(fn):
    """Operators take and return ``SparseTensor``; their bodies work on the wrapped torch tensors."""
    import functools

    @functools.wraps(fn)
    def wrapped(*args, **kwargs):
        return wrap(fn(*unwrap(args), **unwrap(kwargs)))
    return wrapped


class SparseTensor:
    def __init__(self, t):
        self._t = t

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        return wrap(func(*unwrap(args), **unwrap(kwargs or {})))

    # ---- the reference's interface
    @property
    def shape(self):
        return list(self._t.shape)

    @property
    def dtype(self):
        return self._t.dtype

    @property
    def place(self):
        return self._t.device

    @property
    def stop_gradient(self):
        return not self._t.requires_grad

    @stop_gradient.setter
    def stop_gradient(self, v):
        self._t.requires_grad_(not v)

    @property
    def grad(self):
        return wrap(self._t.grad) if self._t.grad is not None else None

    def is_sparse(self):
        return True

    def is_sparse_coo(self):
        return self._t.layout == torch.sparse_coo

    def is_sparse_csr(self):
        return self._t.layout == torch.sparse_csr

    def is_dense(self):
        return False

    def indices(self):
        t = self._t if self._t.layout == torch.sparse_coo else self._t.to_sparse_coo()
        return as_tensor(t.coalesce().indices() if not t.is_coalesced() and not t.requires_grad else t._indices())

    def values(self):
        if self._t.layout == torch.sparse_csr:
            return as_tensor(self._t.values())
        return as_tensor(self._t.coalesce().values() if not self._t.is_coalesced() and not self._t.requires_grad else self._t._values())

    def crows(self):
        return as_tensor((self._t if self._t.layout == torch.sparse_csr else self._t.to_sparse_csr()).crow_indices())

    def cols(self):
        return as_tensor((self._t if self._t.layout == torch.sparse_csr else self._t.to_sparse_csr()).col_indices())

    def nnz(self):
        return int(self._t._nnz())

    def to_dense(self):
        return as_tensor(self._t.to_dense())

    def to_sparse_coo(self, sparse_dim=None):
        if self._t.layout == torch.sparse_coo:
            return self
        return SparseTensor(self._t.to_sparse_coo())

    def to_sparse_csr(self):
        return self if self._t.layout == torch.sparse_csr else SparseTensor(self._t.to_sparse_csr())

    def coalesce(self):
        return SparseTensor(self._t.coalesce())

    def numpy(self):
        return self._t.to_dense().detach().cpu().numpy()

    def astype(self, dtype):
        return SparseTensor(self._t.to(_dt.to_torch(dtype)))

    def backward(self, grad_tensor=None, retain_graph=False):
        g = unwrap(grad_tensor)
        if g is None:
            g = torch.ones_like(self._t.to_dense()).to_sparse_coo() if self._t.layout == torch.sparse_coo else None
        self._t.backward(g, retain_graph=retain_graph)

    def dim(self):
        return self._t.dim()

    ndim = property(lambda self: self._t.dim())

    def __getattr__(self, name):
        # everything else is answered by the wrapped tensor (layout, device, is_coalesced, requires_grad ...)
        attr = getattr(object.__getattribute__(self, "_t"), name)
        if callable(attr):
            return lambda *a, **k: wrap(attr(*unwrap(a), **unwrap(k)))
        return wrap(attr)

    # ---- arithmetic goes through the operators of paddle.sparse
    def _bin(self, other, op, swap=False):
        from .. import sparse
        a, b = (other, self) if swap else (self, other)
        return getattr(sparse, op)(a, b)

    def __add__(self, o): return self._bin(o, "add")
    def __sub__(self, o): return self._bin(o, "subtract")
    def __mul__(self, o): return self._bin(o, "multiply")
    def __truediv__(self, o): return self._bin(o, "divide")
    def __matmul__(self, o): return self._bin(o, "matmul")

    def __neg__(self):
        from .. import sparse
        return sparse.neg(self)

    def __repr__(self):
        from ..tensor.to_string import format_array, place_str
        t = self._t.detach()
        head = (f"Tensor(shape={list(t.shape)}, dtype=paddle.{_dt.to_name(t.dtype)}, place={place_str(t.device)}, "
                f"stop_gradient={self.stop_gradient},")
        pad = " " * 7
        if t.layout == torch.sparse_csr:
            fields = [("crows", t.crow_indices()), ("cols", t.col_indices()), ("values", t.values())]
        else:
            t = t.coalesce() if not t.is_coalesced() else t
            fields = [("indices", t._indices()), ("values", t._values())]
        lines = [f"{pad}{name}={format_array(v.cpu().numpy(), len(pad) + len(name) + 1)}" for name, v in fields]
        return head + "\n" + ",\n".join(lines) + ")"

    __str__ = __repr__
