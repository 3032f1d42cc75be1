"""Operators whose behaviour in the reference differs from the same-named torch function, written out with the
reference's semantics (argument names, defaults, dtypes of results, tie / edge-case rules).  ``install`` puts them over
the table-driven wrappers in the package root, in ``paddle.tensor`` and on ``Tensor``.  Each docstring names the rule
that differs; the worked examples in the reference's docstrings (python/paddle/tensor/*.py) are the test vectors
(``tests/test_docstring_examples_cpu.py``)."""
from __future__ import annotations

import builtins
import math as _math

import numpy as np
import torch

from .._core import dtype as _dt
from .._core.tensor import Tensor, as_tensor


def _t(x):
    return x if isinstance(x, torch.Tensor) else as_tensor(torch.as_tensor(x))


def _axes(axis, nd):
    if axis is None:
        return None
    if isinstance(axis, torch.Tensor):
        axis = axis.tolist()
    if isinstance(axis, (list, tuple)):
        return [int(a) % nd if nd else 0 for a in axis]
    return int(axis)


# ------------------------------------------------------------------------------------------------------- tensor arrays
def create_array(dtype, initialized_list=None):
    """A tensor array is a Python list in dynamic mode (python/paddle/tensor/array.py:268)."""
    arr = list(initialized_list or [])
    for v in arr:
        if not isinstance(v, torch.Tensor):
            raise TypeError(f"All values in `initialized_list` should be Tensor, but received {type(v)}.")
    return arr


def array_length(array):
    return len(array)


def array_read(array, i):
    return array[int(i)]


def array_write(x, i, array=None):
    i = int(i)
    array = [] if array is None else array
    if i > len(array):
        raise ValueError(f"index {i} is beyond the end of an array of length {len(array)}")
    if i < len(array):
        array[i] = x
    else:
        array.append(x)
    return array


def tensor_array_to_tensor(input, axis=1, use_stack=False, name=None):
    """-> (concatenated or stacked tensor, int32 sizes of the pieces along ``axis``)."""
    xs = list(input)
    out = torch.stack(xs, axis) if use_stack else torch.cat(xs, axis)
    sizes = [1] * len(xs) if use_stack else [int(x.shape[axis]) for x in xs]
    return out, as_tensor(torch.tensor(sizes, dtype=torch.int32))


def create_tensor(dtype, name=None, persistable=False):
    return as_tensor(torch.empty(0, dtype=_dt.to_torch(dtype)))


# ------------------------------------------------------------------------------------------------------------- creation
def assign(x, output=None):
    """Copy of ``x`` (tensor, array, list, scalar; float64 data narrows to float32 as in the reference); with ``output``
    given that tensor takes the value (and shape / dtype) and is returned."""
    if isinstance(x, torch.Tensor):
        val = x.clone()
    else:
        arr = np.asarray(x)
        if arr.dtype == np.float64:
            arr = arr.astype(np.float32)
        val = torch.from_numpy(np.ascontiguousarray(arr))
    if output is None:
        return as_tensor(val)
    with torch.no_grad():
        if tuple(output.shape) != tuple(val.shape) or output.dtype != val.dtype:
            output.data = val.detach().to(output.device)          # the output takes the value's shape and dtype
        else:
            torch.Tensor.copy_(output, val)
    return output


def _memcpy(input, place=None, output=None):
    dev = getattr(place, "device", None) or (torch.device("cpu") if place is None or "cpu" in str(place).lower() else torch.device("cuda"))
    res = _t(input).to(dev)
    if output is not None:
        return assign(res, output)
    return as_tensor(res)


# ---------------------------------------------------------------------------------------------------------------- math
def _shift(x, y, left, is_arithmetic):
    x, y = _t(x), _t(y) if isinstance(y, torch.Tensor) else torch.as_tensor(y, dtype=_t(x).dtype)
    if left:
        return torch.bitwise_left_shift(x, y)
    if is_arithmetic or x.dtype == torch.uint8:
        return torch.bitwise_right_shift(x, y)
    # logical right shift on a signed type: shift the two's-complement bit pattern
    bits = x.element_size() * 8
    wide = x.to(torch.int64) & ((1 << bits) - 1) if bits < 64 else x
    if bits == 64:
        shifted = torch.where(y > 0, (x >> 1 & 0x7FFFFFFFFFFFFFFF) >> (y - 1).clamp(min=0), x)
        return shifted
    out = wide >> y.to(torch.int64)
    half = 1 << (bits - 1)
    return torch.where(out >= half, out - (1 << bits), out).to(x.dtype)


def bitwise_left_shift(x, y, is_arithmetic=True, out=None, name=None):
    return _shift(x, y, True, is_arithmetic)


def bitwise_right_shift(x, y, is_arithmetic=True, out=None, name=None):
    """``is_arithmetic=False`` shifts zeros in from the left also for negative values."""
    return _shift(x, y, False, is_arithmetic)


def prod(x, axis=None, keepdim=False, dtype=None, name=None):
    """``dtype`` converts the input BEFORE multiplying (so 0.2 * 0.3 as int64 is 0)."""
    x = _t(x)
    if dtype is not None:
        x = x.to(_dt.to_torch(dtype))
    ax = _axes(axis, x.dim())
    if ax is None or (isinstance(ax, list) and not ax):
        out = torch.prod(x)
        return out.reshape([1] * x.dim()) if keepdim else out
    for a in sorted(ax if isinstance(ax, list) else [ax], reverse=True):
        x = torch.prod(x, a, keepdim=keepdim)
    return x


def digamma(x, name=None):
    """psi(0) is nan here (the reference's kernel), where torch returns -inf."""
    x = _t(x)
    return torch.where(x == 0, torch.full_like(x, float("nan")), torch.digamma(x))


def frexp(x, name=None):
    """The exponent comes back in the floating dtype of ``x``."""
    m, e = torch.frexp(_t(x))
    return m, e.to(m.dtype)


def _tie_mask_grad_reduce(x, axis, keepdim, largest, even):
    """max / min style reduction; ``even`` splits the gradient between tied extrema (amax / amin), otherwise the
    gradient goes to every tied element in full (max / min of the reference)."""
    x = _t(x)
    if not (x.requires_grad and torch.is_grad_enabled()):
        # no gradient to shape: straight to torch (also covers bool / integer inputs)
        if axis is None or (isinstance(axis, (list, tuple)) and len(axis) == 0):
            out = torch.max(x) if largest else torch.min(x)
            return out.reshape([1] * x.dim()) if keepdim else out
        if isinstance(axis, torch.Tensor):
            axis = axis.tolist()
        return (torch.amax if largest else torch.amin)(x, axis if isinstance(axis, int) else tuple(axis), keepdim=keepdim)
    ax = _axes(axis, x.dim())
    dims = list(range(x.dim())) if ax is None else (ax if isinstance(ax, list) else [ax])
    dims = list(dims) or list(range(x.dim()))
    val = (torch.amax if largest else torch.amin)(x, dims, keepdim=True) if x.dim() else x
    if even or not (x.requires_grad and torch.is_grad_enabled()):
        out = val
    else:
        mask = (x == val.detach()).to(x.dtype)
        # value of the extremum, gradient 1 for every tied position
        out = val.detach() + (x * mask).sum(dims, keepdim=True) - (x.detach() * mask).sum(dims, keepdim=True)
    if not keepdim and x.dim():
        out = out.squeeze(dims) if dims else out
    return out


def max(x, axis=None, keepdim=False, name=None):
    """Value only (no indices); every tied maximum receives the full gradient."""
    return _tie_mask_grad_reduce(x, axis, keepdim, True, False)


def min(x, axis=None, keepdim=False, name=None):
    return _tie_mask_grad_reduce(x, axis, keepdim, False, False)


def amax(x, axis=None, keepdim=False, name=None):
    """Tied maxima share the gradient evenly."""
    return _tie_mask_grad_reduce(x, axis, keepdim, True, True)


def amin(x, axis=None, keepdim=False, name=None):
    return _tie_mask_grad_reduce(x, axis, keepdim, False, True)


def median(x, axis=None, keepdim=False, mode="avg", name=None):
    """``mode="avg"`` (default): an even count gives the mean of the two middle values; ``mode="min"`` the lower one,
    together with its index when ``axis`` is given."""
    x = _t(x)
    if mode not in ("avg", "min"):
        raise ValueError(f"Mode {mode} is not supported. Must be avg or min.")
    if axis is None:
        flat = x.reshape(-1)
        n = flat.numel()
        s = torch.sort(flat).values
        if mode == "avg":
            out = (s[(n - 1) // 2].to(torch.float64 if x.dtype == torch.float64 else torch.float32) + s[n // 2]) / 2
            out = out.to(x.dtype if x.dtype.is_floating_point else torch.float32)
        else:
            out = s[(n - 1) // 2]
        return out.reshape([1] * x.dim()) if keepdim else out
    axis = int(axis) % x.dim() if x.dim() else 0
    n = x.shape[axis]
    s, idx = torch.sort(x, dim=axis, stable=True)
    lo = s.select(axis, (n - 1) // 2)
    # a slice holding NaN has median NaN, found at the first NaN
    nan_mask = torch.isnan(x) if x.dtype.is_floating_point else None
    has_nan = nan_mask.any(axis) if nan_mask is not None else None
    if mode == "min":
        i = idx.select(axis, (n - 1) // 2)
        if has_nan is not None:
            lo = torch.where(has_nan, torch.full_like(lo, float("nan")), lo)
            i = torch.where(has_nan, nan_mask.to(torch.int8).argmax(axis), i)
        return (torch.unsqueeze(lo, axis), torch.unsqueeze(i, axis)) if keepdim else (lo, i)
    hi = s.select(axis, n // 2)
    ft = x.dtype if x.dtype.is_floating_point else torch.float32
    out = (lo.to(ft) + hi.to(ft)) / 2
    if has_nan is not None:
        out = torch.where(has_nan, torch.full_like(out, float("nan")), out)
    return torch.unsqueeze(out, axis) if keepdim else out


def nanmedian(x, axis=None, keepdim=False, mode="avg", name=None):
    """Median ignoring NaN; ``avg`` / ``min`` as in ``median``; an all-NaN slice gives NaN."""
    x = _t(x)
    if axis is None or isinstance(axis, (list, tuple)):
        dims = list(range(x.dim())) if axis is None else [a % x.dim() for a in axis]
        keep = [d for d in range(x.dim()) if d not in dims]
        y = x.permute(keep + dims).reshape([x.shape[d] for d in keep] + [-1])
        out = nanmedian(y, -1, False, mode)
        out, idx = out if isinstance(out, tuple) else (out, None)
        if keepdim:
            shape = [1 if d in dims else x.shape[d] for d in range(x.dim())]
            out = out.reshape(shape)
            idx = idx.reshape(shape) if idx is not None else None
        return out
    axis = int(axis) % x.dim()
    n_valid = (~torch.isnan(x)).sum(axis)
    s, idx = torch.sort(torch.where(torch.isnan(x), torch.full_like(x, float("inf")), x), dim=axis, stable=True)
    lo_i = ((n_valid - 1).clamp(min=0) // 2).unsqueeze(axis)
    hi_i = (n_valid.clamp(min=1) // 2).clamp(max=x.shape[axis] - 1).unsqueeze(axis)
    lo, hi = s.gather(axis, lo_i), s.gather(axis, hi_i)
    nanv = torch.full_like(lo, float("nan"))
    if mode == "min":
        out = torch.where(n_valid.unsqueeze(axis) == 0, nanv, lo)
        ind = idx.gather(axis, lo_i)
        return (out, ind) if keepdim else (out.squeeze(axis), ind.squeeze(axis))
    out = torch.where(n_valid.unsqueeze(axis) == 0, nanv, (lo + hi) / 2)
    return out if keepdim else out.squeeze(axis)


def _quantile(x, q, axis, keepdim, interpolation, ignore_nan):
    x = _t(x)
    scalar_q = not isinstance(q, (list, tuple, torch.Tensor)) or (isinstance(q, torch.Tensor) and q.dim() == 0)
    qs = torch.as_tensor(q, dtype=torch.float64).reshape(-1)
    if bool(((qs < 0) | (qs > 1)).any()):
        raise ValueError("q should be in range [0, 1]")
    work = x.to(torch.float64 if x.dtype == torch.float64 else torch.float32)
    if axis is None:
        dims = list(range(x.dim()))
    else:
        dims = [a % x.dim() for a in (axis if isinstance(axis, (list, tuple)) else [axis])]
    keep = [d for d in range(x.dim()) if d not in dims]
    y = work.permute(keep + dims).reshape([x.shape[d] for d in keep] + [-1])
    fn = torch.nanquantile if ignore_nan else torch.quantile
    out = fn(y, qs.to(y.dtype), dim=-1, keepdim=False, interpolation=interpolation)          # [len(q), *keep]
    if keepdim:
        out = out.reshape([len(qs)] + [1 if d in dims else x.shape[d] for d in range(x.dim())])
    return out[0] if scalar_q else out


def quantile(x, q, axis=None, keepdim=False, interpolation="linear", name=None):
    """``axis`` may be a list (those dims are flattened together); the result is float32 / float64."""
    return _quantile(x, q, axis, keepdim, interpolation, False)


def nanquantile(x, q, axis=None, keepdim=False, interpolation="linear", name=None):
    return _quantile(x, q, axis, keepdim, interpolation, True)


# -------------------------------------------------------------------------------------------------------- manipulation
def reshape(x, shape, name=None):
    """A 0 in ``shape`` copies the input's dim at that position; -1 is inferred."""
    x = _t(x)
    if isinstance(shape, torch.Tensor):
        shape = shape.tolist()
    shape = [int(s.item()) if isinstance(s, torch.Tensor) else int(s) for s in shape]
    if 0 in shape and x.numel() > 0:
        # with elements present a literal 0 could never be a valid extent: it copies the input's dim (the reference's
        # rule); an empty input keeps torch's reading of 0 as an empty extent
        shape = [x.shape[i] if (s == 0 and i < x.dim()) else s for i, s in enumerate(shape)]
    return torch.reshape(x, shape)


def expand_as(x, y, name=None):
    x = _t(x)
    return torch.Tensor.expand(x, list(y.shape))


def tensordot(x, y, axes=2, name=None):
    """``axes``: an int n (last n dims of x with first n of y), a flat list (the same dims of both), or a pair of lists;
    a shorter list of the pair is extended by the other's tail (the reference's rule)."""
    x, y = _t(x), _t(y)
    if isinstance(axes, torch.Tensor):
        axes = axes.tolist()
    if isinstance(axes, int):
        return torch.tensordot(x, y, dims=axes)
    axes = list(axes)
    if not axes:
        return torch.tensordot(x, y, dims=0)
    if isinstance(axes[0], (list, tuple, torch.Tensor)):
        ax = [list(a.tolist() if isinstance(a, torch.Tensor) else a) for a in axes]
        a_x = ax[0]
        a_y = ax[1] if len(ax) > 1 else list(ax[0])
    else:
        a_x, a_y = list(axes), list(axes)
    if len(a_x) < len(a_y):
        a_x = a_x + a_y[len(a_x):]
    elif len(a_y) < len(a_x):
        a_y = a_y + a_x[len(a_y):]
    return torch.tensordot(x, y, dims=(a_x, a_y))


def crop(x, shape=None, offsets=None, name=None):
    """Slice ``shape`` elements starting at ``offsets`` (zeros by default); -1 in ``shape`` keeps everything from the
    offset on; both may be lists (of ints or 0-d tensors) or tensors."""
    x = _t(x)

    def ints(v, default):
        if v is None:
            return default
        if isinstance(v, torch.Tensor):
            return [int(i) for i in v.tolist()]
        return [int(i.item()) if isinstance(i, torch.Tensor) else int(i) for i in v]
    offsets = ints(offsets, [0] * x.dim())
    shape = ints(shape, list(x.shape))
    idx = tuple(builtins.slice(o, None if s == -1 else o + s) for o, s in zip(offsets, shape))
    return x[idx]


def scatter(x, index, updates, overwrite=True, name=None):
    """Rows of ``updates`` go to rows ``index`` of a copy of ``x``.  ``overwrite=False``: the target rows are zeroed first
    and repeated indices accumulate."""
    x, updates = _t(x), _t(updates)
    index = _t(index).to(torch.int64).reshape(-1)
    out = x.clone()
    if overwrite:
        out[index] = updates.to(x.dtype)
        return out
    out[index] = 0
    return torch.index_add(out, 0, index, updates.to(x.dtype))


def index_fill(x, index, axis, value, name=None):
    x = _t(x)
    if isinstance(value, torch.Tensor):
        value = value.item()
    return torch.index_fill(x, int(axis), _t(index).to(torch.int64), value)


def index_fill_(x, index, axis, value, name=None):
    if isinstance(value, torch.Tensor):
        value = value.item()
    return torch.Tensor.index_fill_(x, int(axis), _t(index).to(torch.int64), value)


def fill_diagonal_tensor(x, y, offset=0, dim1=0, dim2=1, name=None):
    """A copy of ``x`` whose diagonal (of the planes ``dim1`` x ``dim2``) holds ``y`` (last dim of ``y`` runs along it)."""
    out = _t(x).clone()
    torch.diagonal(out, offset, dim1, dim2).copy_(_t(y).to(out.dtype))
    return out


def fill_diagonal_tensor_(x, y, offset=0, dim1=0, dim2=1, name=None):
    with torch.no_grad():
        torch.diagonal(x, offset, dim1, dim2).copy_(_t(y).to(x.dtype))
    return x


def unique(x, return_index=False, return_inverse=False, return_counts=False, axis=None, dtype="int64", name=None):
    """Sorted unique values; ``return_index`` gives the FIRST occurrence of each; index dtypes follow ``dtype``."""
    x = _t(x)
    it = _dt.to_torch(dtype)
    if axis is None:
        flat = x.reshape(-1)
        vals, inv, counts = torch.unique(flat, sorted=True, return_inverse=True, return_counts=True)
        outs = [vals]
        if return_index:
            first = torch.full((vals.numel(),), flat.numel(), dtype=torch.int64)
            first.scatter_reduce_(0, inv, torch.arange(flat.numel()), reduce="amin")
            outs.append(first.to(it))
        if return_inverse:
            outs.append(inv.to(it))
        if return_counts:
            outs.append(counts.to(it))
        return outs[0] if len(outs) == 1 else tuple(outs)
    vals, inv, counts = torch.unique(x, sorted=True, return_inverse=True, return_counts=True, dim=axis)
    outs = [vals]
    if return_index:
        n = x.shape[axis]
        first = torch.full((vals.shape[axis],), n, dtype=torch.int64)
        first.scatter_reduce_(0, inv, torch.arange(n), reduce="amin")
        outs.append(first.to(it))
    if return_inverse:
        outs.append(inv.to(it))
    if return_counts:
        outs.append(counts.to(it))
    return outs[0] if len(outs) == 1 else tuple(outs)


def nonzero(x, as_tuple=False):
    """``as_tuple=True`` returns one [n, 1] column per dim."""
    x = _t(x)
    if not as_tuple:
        return torch.nonzero(x)
    return tuple(c.reshape(-1, 1) for c in torch.nonzero(x, as_tuple=True))


def put_along_axis(arr, indices, values, axis, reduce="assign", include_self=True, broadcast=True, name=None):
    """Scatter ``values`` along ``axis``; with ``broadcast`` the index (and values) are first broadcast against ``arr`` on
    the other dims.  ``reduce``: assign, add, mul / multiply, mean, amin, amax."""
    arr, indices = _t(arr), _t(indices).to(torch.int64)
    values = values if isinstance(values, torch.Tensor) else torch.as_tensor(values, dtype=arr.dtype)
    values = values.to(arr.dtype)
    axis = int(axis) % arr.dim()
    if broadcast:
        tgt = list(arr.shape)
        tgt[axis] = indices.shape[axis] if indices.dim() == arr.dim() else 1
        if indices.dim() == arr.dim():
            indices = torch.broadcast_to(indices, tgt)
        values = torch.broadcast_to(values, list(indices.shape))
    elif values.dim() == 0:
        values = torch.broadcast_to(values, list(indices.shape))
    if reduce == "assign":
        return torch.scatter(arr, axis, indices, values)
    if reduce == "add":
        return torch.scatter_add(arr, axis, indices, values) if include_self else \
            torch.scatter_reduce(arr, axis, indices, values, "sum", include_self=False)
    red = {"mul": "prod", "multiply": "prod", "mean": "mean", "amin": "amin", "amax": "amax"}.get(reduce)
    if red is None:
        raise ValueError(f"unsupported reduce {reduce!r}")
    return torch.scatter_reduce(arr, axis, indices, values, red, include_self=include_self)


def histogramdd(x, bins=10, ranges=None, density=False, weights=None, name=None):
    """-> (histogram, list of bin-edge tensors); ``ranges`` is a flat [lo0, hi0, lo1, hi1, ...] sequence."""
    x = _t(x)
    kw = {}
    if ranges is not None:
        kw["range"] = [float(r) for r in ranges]
    if isinstance(bins, (list, tuple)) and bins and isinstance(bins[0], torch.Tensor):
        bins = [b.to(x.dtype) for b in bins]
    res = torch.histogramdd(x, bins=bins, weight=None if weights is None else _t(weights), density=bool(density), **kw)
    return as_tensor(res.hist), [as_tensor(e) for e in res.bin_edges]


# -------------------------------------------------------------------------------------------------------------- linalg
def matrix_rank(x, tol=None, hermitian=False, atol=None, rtol=None, name=None):
    x = _t(x)
    if tol is not None:
        tol_t = tol if isinstance(tol, torch.Tensor) else torch.tensor(float(tol), dtype=x.dtype if x.dtype.is_floating_point else torch.float32)
        s = torch.linalg.eigvalsh(x).abs() if hermitian else torch.linalg.svdvals(x)
        return (s > tol_t.unsqueeze(-1) if tol_t.dim() else s > tol_t).sum(-1).to(torch.int32)
    kw = {}
    if atol is not None:
        kw["atol"] = atol if isinstance(atol, torch.Tensor) else torch.tensor(float(atol))
    if rtol is not None:
        kw["rtol"] = rtol if isinstance(rtol, torch.Tensor) else torch.tensor(float(rtol))
    return torch.linalg.matrix_rank(x, hermitian=hermitian, **kw).to(torch.int32)


def lu(x, pivot=True, get_infos=False, name=None):
    """-> (LU, int32 pivots (1-based) [, int32 info per matrix])."""
    lu_, piv, info = torch.linalg.lu_factor_ex(_t(x), pivot=pivot)
    info = info.to(torch.int32)
    return (lu_, piv.to(torch.int32), info) if get_infos else (lu_, piv.to(torch.int32))


def lstsq(x, y, rcond=None, driver=None, name=None):
    """-> (solution, residuals, int32 rank, singular values)."""
    x, y = _t(x), _t(y)
    if driver is None:
        driver = "gelsy" if x.device.type == "cpu" else "gels"
    r = torch.linalg.lstsq(x, y, rcond=rcond, driver=driver)
    return r.solution, r.residuals, r.rank.to(torch.int32), r.singular_values


# -------------------------------------------------------------------------------------------------------------- random
def bernoulli_(x, p=0.5, name=None):
    """Fill ``x`` in place with draws of probability ``p`` (a float or a tensor broadcastable to ``x``)."""
    with torch.no_grad():
        if isinstance(p, torch.Tensor):                   # uniform draw below p; p outside [0, 1] saturates
            u = torch.rand(x.shape, dtype=x.dtype if x.dtype.is_floating_point else torch.float32, device=x.device)
            return torch.Tensor.copy_(x, (u < torch.broadcast_to(p.to(u.dtype), x.shape)).to(x.dtype))
        return torch.Tensor.bernoulli_(x, builtins.min(builtins.max(float(p), 0.0), 1.0))


def log_normal(mean=1.0, std=2.0, shape=None, dtype=None, name=None):
    """exp of a normal sample; ``mean`` / ``std`` (of the underlying normal) may be tensors, which then give the shape."""
    dt = _dt.to_torch(dtype) if dtype is not None else torch.get_default_dtype()
    if isinstance(mean, torch.Tensor) or isinstance(std, torch.Tensor):
        m = mean if isinstance(mean, torch.Tensor) else torch.tensor(float(mean), dtype=dt)
        s = std if isinstance(std, torch.Tensor) else torch.tensor(float(std), dtype=dt)
        m, s = torch.broadcast_tensors(m, s)
        return as_tensor(torch.exp(torch.normal(m.to(dt), s.to(dt))))
    shape = [1] if shape is None else [int(v) for v in (shape.tolist() if isinstance(shape, torch.Tensor) else shape)]
    return as_tensor(torch.exp(torch.normal(float(mean), float(std), shape, dtype=dt)))


def gaussian_(x, mean=0.0, std=1.0, seed=0, name=None):
    with torch.no_grad():
        return torch.Tensor.normal_(x, float(mean), float(std))


def round(x, decimals=0, name=None):
    """Halves round away from zero (-0.5 -> -1, 2.5 -> 3), unlike torch's round-half-to-even."""
    x = _t(x)
    if not x.dtype.is_floating_point:
        return x.clone()
    scale = 10.0 ** int(decimals)
    y = x * scale if decimals else x
    out = torch.copysign(torch.floor(y.abs() + 0.5), y)
    return out / scale if decimals else out


def round_(x, decimals=0, name=None):
    with torch.no_grad():
        return torch.Tensor.copy_(x, round(x, decimals))


# ----------------------------------------------------------------------------------------------------- Tensor methods
class _CallableTensor(Tensor):
    """``x.real`` is an attribute in torch and a method in the reference: the attribute's value can also be called."""

    def __call__(self, name=None):
        return self


def _field(self, which):
    plain = self.as_subclass(torch.Tensor)
    if which == "imag" and not plain.is_complex():
        raise RuntimeError("imag is not implemented for tensors with non-complex dtypes.")
    val = getattr(plain, which)
    return val.as_subclass(_CallableTensor)


def _to_sparse_coo(self, sparse_dim=None):
    """COO form with the first ``sparse_dim`` dims indexed (all dims by default)."""
    plain = self.detach().as_subclass(torch.Tensor) if not self.requires_grad else self.as_subclass(torch.Tensor)
    from ..sparse.tensor import SparseTensor
    return SparseTensor(plain.to_sparse(sparse_dim if sparse_dim is not None else plain.dim()))


def _to_sparse_csr(self):
    from ..sparse.tensor import SparseTensor
    plain = self.detach().as_subclass(torch.Tensor) if not self.requires_grad else self.as_subclass(torch.Tensor)
    return SparseTensor(plain.to_sparse_csr())


def _reshape_method(self, *shape, **kw):
    if "shape" in kw:
        shape = (kw["shape"],)
    if len(shape) == 1 and isinstance(shape[0], (list, tuple, torch.Size, torch.Tensor)):
        shape = shape[0]
    if not isinstance(shape, torch.Tensor):
        try:
            if 0 not in shape:                                       # the common case goes straight to torch
                return torch.Tensor.reshape(self, tuple(shape))
        except (TypeError, RuntimeError):
            pass
    return reshape(self, list(shape) if not isinstance(shape, torch.Tensor) else shape)


def _set_(self, source=None, shape=None, stride=None, offset=0, name=None):
    """Share ``source``'s storage (no copy), optionally viewed with ``shape`` / ``stride`` / byte ``offset``; without a
    source the tensor becomes empty."""
    with torch.no_grad():
        if source is None:
            return torch.Tensor.set_(self, torch.empty(0, dtype=self.dtype, device=self.device))
        if shape is None and stride is None and not offset:
            return torch.Tensor.set_(self, source.detach())
        shape = list(source.shape) if shape is None else [int(v) for v in shape]
        if stride is None:
            stride, acc = [], 1
            for d in reversed(shape):
                stride.insert(0, acc)
                acc *= d
        return torch.Tensor.set_(self, source.detach().untyped_storage(), int(offset) // source.element_size(), shape, [int(v) for v in stride])


def _retain_grads(self):
    """Keep ``.grad`` of a non-leaf tensor after backward."""
    if self.requires_grad and not self.is_leaf:
        torch.Tensor.retain_grad(self)


def _is_shared_buffer_with(self, other):
    return self.untyped_storage().data_ptr() == other.untyped_storage().data_ptr()


def _resize_(self, shape, fill_zero=False, name=None):
    """In-place resize keeping the leading elements; ``fill_zero`` zeroes newly exposed elements."""
    old = self.numel()
    shape = [int(s) for s in shape]
    with torch.no_grad():
        torch.Tensor.resize_(self, shape)
        if fill_zero and self.numel() > old:
            self.reshape(-1)[old:].zero_()
    return self


_FUNCTIONS = ["create_array", "array_length", "array_read", "array_write", "tensor_array_to_tensor", "create_tensor", "assign", "_memcpy",
              "bitwise_left_shift", "bitwise_right_shift", "prod", "digamma", "frexp", "max", "min", "amax", "amin", "median", "nanmedian", "quantile",
              "nanquantile", "reshape", "expand_as", "tensordot", "crop", "scatter", "index_fill", "index_fill_", "fill_diagonal_tensor",
              "fill_diagonal_tensor_", "unique", "nonzero", "put_along_axis", "histogramdd", "matrix_rank", "lu", "lstsq", "bernoulli_", "log_normal", "gaussian_", "round", "round_"]
_METHODS = ["bitwise_left_shift", "bitwise_right_shift", "prod", "digamma", "frexp", "max", "min", "amax", "amin", "median", "nanmedian", "quantile",
            "nanquantile", "expand_as", "tensordot", "crop", "scatter", "index_fill", "index_fill_", "fill_diagonal_tensor",
            "fill_diagonal_tensor_", "unique", "nonzero", "put_along_axis", "matrix_rank", "bernoulli_"]


def _wrapping(fn):
    """Results built from raw torch tensors come back as this package's Tensor."""
    import functools

    def conv(o):
        if isinstance(o, torch.Tensor) and not isinstance(o, Tensor):
            return as_tensor(o)
        if isinstance(o, tuple):
            return tuple(conv(v) for v in o)
        if isinstance(o, list):
            return [conv(v) for v in o]
        return o

    @functools.wraps(fn)
    def wrapped(*a, **k):
        return conv(fn(*a, **k))
    return wrapped


def install(root_namespace):
    """Put the functions above over the generic wrappers: package root, ``paddle.tensor`` and its sub-modules that
    define the same name, ``paddle.linalg``, and ``Tensor`` methods."""
    import importlib
    import sys
    g = globals()
    pkg = __name__.rsplit(".", 1)[0]
    mods = [sys.modules[pkg]] + [importlib.import_module(f"{pkg}.{m}") for m in ("math", "manipulation", "creation", "linalg", "random", "extras")]
    try:
        mods.append(importlib.import_module(pkg.rsplit(".", 1)[0] + ".linalg"))
    except ImportError:
        pass
    for name in _FUNCTIONS:
        fn = g[name] = _wrapping(g[name]) if not getattr(g[name], "__wrapped__", None) else g[name]
        root_namespace[name] = fn
        setattr(mods[0], name, fn)
        for m in mods[1:]:
            if hasattr(m, name):
                setattr(m, name, fn)
    arr_mod = type(sys)("array")
    arr_mod.__name__ = pkg + ".array"
    for name in ("create_array", "array_length", "array_read", "array_write", "tensor_array_to_tensor"):
        setattr(arr_mod, name, g[name])
    sys.modules[arr_mod.__name__] = arr_mod
    mods[0].array = arr_mod
    setattr(importlib.import_module(f"{pkg}.random"), "gaussian_", gaussian_)
    setattr(importlib.import_module(f"{pkg}.manipulation"), "tensor_array_to_tensor", tensor_array_to_tensor)
    for name in _METHODS:
        setattr(Tensor, name, g[name])
    Tensor.real = property(lambda self: _field(self, "real"))
    Tensor.imag = property(lambda self: _field(self, "imag"))
    Tensor.to_sparse_coo = _to_sparse_coo
    Tensor.to_sparse_csr = _to_sparse_csr
    Tensor.reshape = _reshape_method
    Tensor.set_ = _set_
    Tensor.round = round
    Tensor.round_ = round_
    Tensor.retain_grads = _retain_grads
    Tensor._is_shared_buffer_with = _is_shared_buffer_with
    Tensor.resize_ = _resize_
