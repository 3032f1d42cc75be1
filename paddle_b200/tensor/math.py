"""Math API (python/paddle/tensor/math.py, ops.py, stat.py, logic.py, search.py in the reference).
Thin wrappers giving Paddle's argument names (``x``, ``y``, ``axis``, ``keepdim``) over torch ops."""
from __future__ import annotations

import builtins
import sys

import numpy as np
import torch

from .._core import dtype as _dt
from .._core.tensor import Tensor, as_tensor, to_tensor

_this = sys.modules[__name__]


def _t(x):
    return x if isinstance(x, torch.Tensor) else to_tensor(x)


# ------------------------------------------------------------------ table-driven unary / binary
_UNARY = {
    "abs": torch.abs, "acos": torch.acos, "asin": torch.asin, "atan": torch.atan, "acosh": torch.acosh,
    "asinh": torch.asinh, "atanh": torch.atanh, "ceil": torch.ceil, "cos": torch.cos, "cosh": torch.cosh,
    "exp": torch.exp, "expm1": torch.expm1, "floor": torch.floor, "log": torch.log, "log2": torch.log2,
    "log10": torch.log10, "log1p": torch.log1p, "reciprocal": torch.reciprocal, "round": torch.round,
    "rsqrt": torch.rsqrt, "sigmoid": torch.sigmoid, "sign": torch.sign, "sin": torch.sin, "sinh": torch.sinh,
    "sqrt": torch.sqrt, "square": torch.square, "tan": torch.tan, "tanh": torch.tanh, "erf": torch.erf,
    "erfinv": torch.erfinv, "lgamma": torch.lgamma, "digamma": torch.digamma, "trunc": torch.trunc,
    "frac": torch.frac, "neg": torch.neg, "isnan": torch.isnan, "isinf": torch.isinf, "isfinite": torch.isfinite,
    "logical_not": torch.logical_not, "bitwise_not": torch.bitwise_not, "angle": torch.angle, "conj": torch.conj,
    "real": torch.real, "imag": torch.imag, "i0": torch.i0, "sgn": torch.sgn, "exp2": torch.exp2,
    "logit": torch.logit, "deg2rad": torch.deg2rad, "rad2deg": torch.rad2deg, "signbit": torch.signbit,
    "positive": torch.positive, "negative": torch.neg, "isreal": torch.isreal,
}
for _n, _f in _UNARY.items():
    def _mk(f):
        def op(x, name=None):
            return f(_t(x))
        return op
    setattr(_this, _n, _mk(_f))
    getattr(_this, _n).__name__ = _n

_BINARY = {
    "add": torch.add, "subtract": torch.sub, "multiply": torch.mul, "divide": torch.true_divide,
    "maximum": torch.maximum, "minimum": torch.minimum, "fmax": torch.fmax, "fmin": torch.fmin,
    "remainder": torch.remainder, "mod": torch.remainder, "floor_mod": torch.remainder,
    "atan2": torch.atan2, "hypot": torch.hypot, "logaddexp": torch.logaddexp, "heaviside": torch.heaviside,
    "equal": torch.eq, "not_equal": torch.ne, "greater_than": torch.gt, "greater_equal": torch.ge,
    "less_than": torch.lt, "less_equal": torch.le, "logical_and": torch.logical_and,
    "logical_or": torch.logical_or, "logical_xor": torch.logical_xor, "bitwise_and": torch.bitwise_and,
    "bitwise_or": torch.bitwise_or, "bitwise_xor": torch.bitwise_xor, "gcd": torch.gcd, "lcm": torch.lcm,
    "copysign": torch.copysign, "nextafter": torch.nextafter, "ldexp": torch.ldexp,
    "bitwise_left_shift": torch.bitwise_left_shift, "bitwise_right_shift": torch.bitwise_right_shift,
}
for _n, _f in _BINARY.items():
    def _mk2(f):
        def op(x, y, name=None):
            x = _t(x)
            if not isinstance(y, torch.Tensor):
                y = torch.as_tensor(y, device=x.device, dtype=x.dtype if isinstance(y, float) or x.dtype.is_floating_point else None)
            return f(x, y)
        return op
    setattr(_this, _n, _mk2(_f))
    getattr(_this, _n).__name__ = _n


def floor_divide(x, y, name=None):
    return torch.div(_t(x), y, rounding_mode="floor")


def pow(x, y, name=None):
    return torch.pow(_t(x), y)


def scale(x, scale=1.0, bias=0.0, bias_after_scale=True, act=None, name=None):
    return x * scale + bias if bias_after_scale else (x + bias) * scale


def clip(x, min=None, max=None, name=None):
    return torch.clamp(x, min=min, max=max)


def lerp(x, y, weight, name=None):
    return torch.lerp(x, y, weight)


def addmm(input, x, y, beta=1.0, alpha=1.0, name=None):
    return torch.addmm(input, x, y, beta=beta, alpha=alpha)


def add_n(inputs, name=None):
    if isinstance(inputs, torch.Tensor):
        return inputs
    r = inputs[0]
    for t in inputs[1:]:
        r = r + t
    return r


def stanh(x, scale_a=0.67, scale_b=1.7159, name=None):
    return scale_b * torch.tanh(scale_a * x)


def multiplex(inputs, index, name=None):
    st = torch.stack(list(inputs), 0)
    idx = index.reshape(-1).long()
    return st[idx, torch.arange(st.shape[1], device=st.device)]


def nan_to_num(x, nan=0.0, posinf=None, neginf=None, name=None):
    return torch.nan_to_num(x, nan, posinf, neginf)


def isclose(x, y, rtol=1e-5, atol=1e-8, equal_nan=False, name=None):
    return torch.isclose(x, y, rtol, atol, equal_nan)


def allclose(x, y, rtol=1e-5, atol=1e-8, equal_nan=False, name=None):
    return as_tensor(torch.tensor(torch.allclose(x, y, rtol, atol, equal_nan)))


def equal_all(x, y, name=None):
    return as_tensor(torch.tensor(x.shape == y.shape and bool(torch.equal(x, y))))


def is_empty(x, name=None):
    return as_tensor(torch.tensor(torch.Tensor.numel(x) == 0))


def is_tensor(x):
    return isinstance(x, torch.Tensor)


def is_complex(x):
    return x.is_complex()


def is_floating_point(x):
    return x.is_floating_point()


def is_integer(x):
    return not x.is_floating_point() and not x.is_complex() and x.dtype != torch.bool


# ------------------------------------------------------------------ reductions
def _axis(axis):
    if isinstance(axis, torch.Tensor):
        axis = axis.tolist()
    if isinstance(axis, (list, tuple)):
        return tuple(int(a) for a in axis)
    return axis


def sum(x, axis=None, dtype=None, keepdim=False, name=None):
    return Tensor.sum(_t(x).as_subclass(Tensor), _axis(axis), dtype, keepdim)


def mean(x, axis=None, keepdim=False, name=None):
    return Tensor.mean(as_tensor(_t(x)), _axis(axis), keepdim)


def prod(x, axis=None, keepdim=False, dtype=None, name=None):
    return Tensor.prod(as_tensor(x), _axis(axis), keepdim, dtype)


def max(x, axis=None, keepdim=False, name=None):
    return Tensor.max(as_tensor(x), _axis(axis), keepdim)


def min(x, axis=None, keepdim=False, name=None):
    return Tensor.min(as_tensor(x), _axis(axis), keepdim)


amax, amin = max, min


def all(x, axis=None, keepdim=False, name=None):
    return Tensor.all(as_tensor(x), _axis(axis), keepdim)


def any(x, axis=None, keepdim=False, name=None):
    return Tensor.any(as_tensor(x), _axis(axis), keepdim)


def std(x, axis=None, unbiased=True, keepdim=False, name=None):
    return torch.std(x, dim=_axis(axis), unbiased=unbiased, keepdim=keepdim)


def var(x, axis=None, unbiased=True, keepdim=False, name=None):
    return torch.var(x, dim=_axis(axis), unbiased=unbiased, keepdim=keepdim)


def median(x, axis=None, keepdim=False, mode="avg", name=None):
    if axis is None:
        return torch.quantile(x.float().reshape(-1), 0.5).to(x.dtype) if mode == "avg" else torch.median(x)
    if mode == "avg":
        return torch.quantile(x.float(), 0.5, dim=axis, keepdim=keepdim).to(x.dtype)
    return torch.median(x, dim=axis, keepdim=keepdim).values


def nanmedian(x, axis=None, keepdim=False, name=None):
    return torch.nanmedian(x) if axis is None else torch.nanmedian(x, dim=axis, keepdim=keepdim).values


def quantile(x, q, axis=None, keepdim=False, interpolation="linear", name=None):
    return torch.quantile(x, torch.as_tensor(q, dtype=x.dtype, device=x.device), dim=axis, keepdim=keepdim,
                          interpolation=interpolation)


def nansum(x, axis=None, dtype=None, keepdim=False, name=None):
    return torch.nansum(x, dim=_axis(axis), keepdim=keepdim) if axis is not None else torch.nansum(x)


def nanmean(x, axis=None, keepdim=False, name=None):
    return torch.nanmean(x, dim=_axis(axis), keepdim=keepdim) if axis is not None else torch.nanmean(x)


def logsumexp(x, axis=None, keepdim=False, name=None):
    if axis is None:
        axis = tuple(range(x.dim()))
    return torch.logsumexp(x, dim=_axis(axis), keepdim=keepdim)


def cumsum(x, axis=None, dtype=None, name=None):
    if axis is None:
        x, axis = x.reshape(-1), 0
    return torch.cumsum(x, axis, dtype=_dt.to_torch(dtype))


def cumprod(x, dim=None, dtype=None, name=None):
    if dim is None:
        x, dim = x.reshape(-1), 0
    return torch.cumprod(x, dim, dtype=_dt.to_torch(dtype))


def cummax(x, axis=None, dtype="int64", name=None):
    if axis is None:
        x, axis = x.reshape(-1), 0
    r = torch.cummax(x, axis)
    return r.values, r.indices.to(_dt.to_torch(dtype))


def cummin(x, axis=None, dtype="int64", name=None):
    if axis is None:
        x, axis = x.reshape(-1), 0
    r = torch.cummin(x, axis)
    return r.values, r.indices.to(_dt.to_torch(dtype))


def logcumsumexp(x, axis=None, dtype=None, name=None):
    if axis is None:
        x, axis = x.reshape(-1), 0
    return torch.logcumsumexp(x, axis)


def count_nonzero(x, axis=None, keepdim=False, name=None):
    r = torch.count_nonzero(x, dim=_axis(axis))
    return r.unsqueeze(axis) if keepdim and axis is not None and isinstance(axis, int) else r


def diff(x, n=1, axis=-1, prepend=None, append=None, name=None):
    return torch.diff(x, n, axis, prepend, append)


def trace(x, offset=0, axis1=0, axis2=1, name=None):
    return torch.diagonal(x, offset, axis1, axis2).sum(-1)


def diagonal(x, offset=0, axis1=0, axis2=1, name=None):
    return torch.diagonal(x, offset, axis1, axis2)


def kron(x, y, name=None):
    return torch.kron(x, y)


def inner(x, y, name=None):
    return torch.inner(x, y)


def outer(x, y, name=None):
    return torch.outer(x.reshape(-1), y.reshape(-1))


def increment(x, value=1.0, name=None):
    return x.add_(value)


def renorm(x, p, axis, max_norm):
    return torch.renorm(x, p, axis, max_norm)


def take(x, index, mode="raise", name=None):
    flat = x.reshape(-1)
    n = flat.shape[0]
    idx = index.long()
    if mode == "wrap":
        idx = idx % n
    elif mode == "clip":
        idx = idx.clamp(0, n - 1)
    else:
        idx = torch.where(idx < 0, idx + n, idx)
    return flat[idx]


def frexp(x, name=None):
    return torch.frexp(x)


def trapezoid(y, x=None, dx=None, axis=-1, name=None):
    return torch.trapezoid(y, x, dim=axis) if x is not None else torch.trapezoid(y, dx=dx or 1.0, dim=axis)


def vander(x, n=None, increasing=False, name=None):
    return torch.vander(x, n, increasing)


def histogram(input, bins=100, min=0, max=0, name=None):
    return torch.histc(input.float(), bins, min, max).to(torch.int64)


def bincount(x, weights=None, minlength=0, name=None):
    return torch.bincount(x, weights, minlength)


# ------------------------------------------------------------------ search / sort
def argmax(x, axis=None, keepdim=False, dtype="int64", name=None):
    return torch.argmax(x, dim=axis, keepdim=keepdim).to(_dt.to_torch(dtype))


def argmin(x, axis=None, keepdim=False, dtype="int64", name=None):
    return torch.argmin(x, dim=axis, keepdim=keepdim).to(_dt.to_torch(dtype))


def argsort(x, axis=-1, descending=False, stable=False, name=None):
    return torch.argsort(x, dim=axis, descending=descending, stable=stable)


def sort(x, axis=-1, descending=False, stable=False, name=None):
    return torch.sort(x, dim=axis, descending=descending, stable=stable).values


def topk(x, k, axis=None, largest=True, sorted=True, name=None):
    if isinstance(k, torch.Tensor):
        k = int(k.item())
    r = torch.topk(x, k, dim=-1 if axis is None else axis, largest=largest, sorted=sorted)
    return r.values, r.indices


def kthvalue(x, k, axis=-1, keepdim=False, name=None):
    r = torch.kthvalue(x, k, axis, keepdim)
    return r.values, r.indices


def mode(x, axis=-1, keepdim=False, name=None):
    r = torch.mode(x, axis, keepdim)
    return r.values, r.indices


def where(condition, x=None, y=None, name=None):
    if x is None and y is None:
        return tuple(t.unsqueeze(-1) for t in torch.where(condition))
    if not isinstance(x, torch.Tensor):
        x = torch.as_tensor(x, device=condition.device, dtype=y.dtype if isinstance(y, torch.Tensor) else None)
    if not isinstance(y, torch.Tensor):
        y = torch.as_tensor(y, device=condition.device, dtype=x.dtype)
    return torch.where(condition, x, y)


def nonzero(x, as_tuple=False):
    return torch.nonzero(x, as_tuple=as_tuple)


def masked_select(x, mask, name=None):
    return torch.masked_select(x, mask)


def masked_fill(x, mask, value, name=None):
    return torch.masked_fill(x, mask, value.item() if isinstance(value, torch.Tensor) and value.numel() == 1 else value)


def index_select(x, index, axis=0, name=None):
    return torch.index_select(x, axis, index.reshape(-1))


def index_sample(x, index):
    return torch.gather(x, 1, index)


def searchsorted(sorted_sequence, values, out_int32=False, right=False, name=None):
    return torch.searchsorted(sorted_sequence, values, out_int32=out_int32, right=right)


def bucketize(x, sorted_sequence, out_int32=False, right=False, name=None):
    return torch.bucketize(x, sorted_sequence, out_int32=out_int32, right=right)


def unique(x, return_index=False, return_inverse=False, return_counts=False, axis=None, dtype="int64", name=None):
    if return_index:
        flat = x.reshape(-1) if axis is None else x
        u, inv, cnt = torch.unique(flat, sorted=True, return_inverse=True, return_counts=True, dim=axis)
        first = torch.full((u.shape[0],), inv.numel(), dtype=torch.int64, device=x.device)
        first.scatter_reduce_(0, inv.reshape(-1), torch.arange(inv.numel(), device=x.device), reduce="amin")
        out = [u, first]
        if return_inverse:
            out.append(inv)
        if return_counts:
            out.append(cnt)
        return tuple(out)
    r = torch.unique(x, sorted=True, return_inverse=return_inverse, return_counts=return_counts, dim=axis)
    return r


def unique_consecutive(x, return_inverse=False, return_counts=False, axis=None, dtype="int64", name=None):
    return torch.unique_consecutive(x, return_inverse, return_counts, axis)
