"""``paddle.sparse`` (python/paddle/sparse/): COO / CSR tensors and operators on them, carried by torch's sparse
layouts.  ``sparse_coo_tensor(indices [ndim, nnz], values, shape)``, ``sparse_csr_tensor(crows, cols, values, shape)``."""
from __future__ import annotations

import torch

from .._core.tensor import as_tensor
from . import nn  # noqa: F401

__all__ = ["sparse_coo_tensor", "sparse_csr_tensor", "sin", "tan", "asin", "atan", "sinh", "tanh", "asinh", "atanh", "sqrt",
           "square", "log1p", "abs", "pow", "cast", "neg", "deg2rad", "rad2deg", "expm1", "mv", "matmul", "masked_matmul",
           "addmm", "add", "subtract", "transpose", "sum", "multiply", "divide", "coalesce", "is_same_shape", "reshape",
           "isnan", "slice", "pca_lowrank", "mask_as"]


from .tensor import SparseTensor, api as _api, unwrap as _unwrap, wrap as _wrap  # noqa: E402


def _p(x):
    x = _unwrap(x)
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def sparse_coo_tensor(indices, values, shape=None, dtype=None, place=None, stop_gradient=True):
    i, v = _p(indices).long(), _p(values)
    if dtype is not None:
        from .._core import dtype as _dt
        v = v.to(_dt.to_torch(dtype))
    t = torch.sparse_coo_tensor(i, v, size=tuple(shape)) if shape is not None else torch.sparse_coo_tensor(i, v)
    t.requires_grad_(not stop_gradient and t.is_floating_point())
    return t


def sparse_csr_tensor(crows, cols, values, shape, dtype=None, place=None, stop_gradient=True):
    v = _p(values)
    if dtype is not None:
        from .._core import dtype as _dt
        v = v.to(_dt.to_torch(dtype))
    return torch.sparse_csr_tensor(_p(crows).long(), _p(cols).long(), v, size=tuple(shape))


def _unary(fn):
    def f(x, name=None):
        if x.layout == torch.sparse_csr:
            return torch.sparse_csr_tensor(x.crow_indices(), x.col_indices(), fn(x.values()), x.shape)
        x = x.coalesce()
        return torch.sparse_coo_tensor(x.indices(), fn(x.values()), x.shape)
    return f


sin, tan, asin, atan, sinh, tanh, asinh, atanh = (_unary(getattr(torch, n)) for n in
                                                  ("sin", "tan", "asin", "atan", "sinh", "tanh", "asinh", "atanh"))
sqrt, square, log1p, abs, neg, expm1, deg2rad, rad2deg, isnan = (
    _unary(getattr(torch, n)) for n in ("sqrt", "square", "log1p", "abs", "neg", "expm1", "deg2rad", "rad2deg", "isnan"))


def pow(x, factor, name=None):
    return _unary(lambda v: torch.pow(v, factor))(x)


def cast(x, index_dtype=None, value_dtype=None, name=None):
    from .._core import dtype as _dt
    x = x.coalesce()
    idx = x.indices().to(_dt.to_torch(index_dtype)) if index_dtype else x.indices()
    val = x.values().to(_dt.to_torch(value_dtype)) if value_dtype else x.values()
    return torch.sparse_coo_tensor(idx.long(), val, x.shape)


def matmul(x, y, name=None):
    out = torch.sparse.mm(x, _p(y)) if x.dim() == 2 else torch.matmul(x.to_dense(), _p(y) if not y.is_sparse else y.to_dense())
    return out if out.is_sparse else as_tensor(out)


def mv(x, vec, name=None):
    return as_tensor(torch.mv(x.to_dense() if x.layout != torch.strided else x, _p(vec)))


def masked_matmul(x, y, mask, name=None):
    dense = torch.matmul(_p(x), _p(y))
    m = mask.to_sparse_coo().coalesce() if mask.layout != torch.sparse_coo else mask.coalesce()
    vals = dense[tuple(m.indices())]
    out = torch.sparse_coo_tensor(m.indices(), vals, m.shape)
    return out.to_sparse_csr() if mask.layout == torch.sparse_csr else out


def addmm(input, x, y, beta=1.0, alpha=1.0, name=None):
    d = lambda t: t.to_dense() if t.layout != torch.strided else _p(t)   # noqa: E731
    return as_tensor(beta * d(input) + alpha * torch.matmul(d(x), d(y)))


def _binary(fn):
    def f(x, y, name=None):
        if isinstance(y, (int, float)):
            return _unary(lambda v: fn(v, y))(x)
        out = fn(x.to_dense(), y.to_dense() if y.layout != torch.strided else _p(y))
        return out.to_sparse_csr() if x.layout == torch.sparse_csr else out.to_sparse_coo()
    return f


add, subtract, multiply, divide = (_binary(f) for f in (torch.add, torch.sub, torch.mul, torch.div))


def transpose(x, perm, name=None):
    return x.to_dense().permute(*perm).to_sparse_coo() if x.layout != torch.sparse_csr else \
        x.to_dense().permute(*perm).to_sparse_csr()


def sum(x, axis=None, dtype=None, keepdim=False, name=None):
    d = x.to_dense()
    if dtype is not None:
        from .._core import dtype as _dt
        d = d.to(_dt.to_torch(dtype))
    if axis is None:                                  # the total comes back as a sparse tensor of shape [1]
        out = d.sum().reshape([1] * d.dim() if keepdim else [1])
    else:
        out = d.sum(axis, keepdim=keepdim)
    return out.to_sparse_csr() if (x.layout == torch.sparse_csr and out.dim() == 2) else out.to_sparse_coo()


def coalesce(x, name=None):
    return x.coalesce()


def is_same_shape(x, y):
    return tuple(x.shape) == tuple(y.shape)


def reshape(x, shape, name=None):
    return x.to_dense().reshape(tuple(shape)).to_sparse_coo()


def slice(x, axes, starts, ends, name=None):
    d = x.to_dense()
    for a, s, e in zip(axes, starts, ends):
        d = d.narrow(a, s, min(e, d.shape[a]) - s)
    return d.to_sparse_coo()


def mask_as(x, mask, name=None):
    m = mask.coalesce() if mask.layout == torch.sparse_coo else mask.to_sparse_coo().coalesce()
    out = torch.sparse_coo_tensor(m.indices(), _p(x)[tuple(m.indices())], m.shape)
    return out.to_sparse_csr() if mask.layout == torch.sparse_csr else out


def pca_lowrank(x, q=None, center=True, niter=2, name=None):
    return tuple(as_tensor(t) for t in torch.pca_lowrank(x.to_dense(), q, center, niter))


# every public operator takes and returns SparseTensor (dense results come back as package tensors)
for _n in list(__all__):
    if callable(globals().get(_n)) and _n != "is_same_shape":
        globals()[_n] = _api(globals()[_n])
is_same_shape = (lambda f: lambda x, y: f(_unwrap(x), _unwrap(y)))(is_same_shape)
del _n
