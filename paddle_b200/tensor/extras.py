"""Remaining names of the top-level tensor API (python/paddle/__init__.py ``__all__``): in-place variants (``x.op_()``
mutates ``x`` and returns it, python/paddle/tensor/math.py ``*_`` wrappers), special functions, splitting / stacking
helpers and dtype information objects."""
from __future__ import annotations

import itertools
import math as _math

import numpy as _np
import torch

from .._core import dtype as _dt
from .._core.tensor import as_tensor

inf, nan, pi, e, newaxis = float("inf"), float("nan"), _math.pi, _math.e, None


def _p(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else x


def _inplace(fn):
    def f(x, *a, name=None, **k):
        r = fn(x, *a, **k)
        with torch.no_grad():
            _p(x).copy_(_p(r).to(x.dtype))
        return x
    return f


def _make_inplace_table():
    from . import linalg as L
    from . import manipulation as MP
    from . import math as M
    names = ["addmm", "t", "cumsum", "cumprod", "logit", "equal", "where", "cos", "tan", "unsqueeze", "logical_and",
             "less_than", "less", "squeeze", "floor_divide", "remainder", "floor_mod", "logical_or", "bitwise_and",
             "bitwise_or", "bitwise_xor", "bitwise_not", "bitwise_invert", "less_equal", "triu", "sin", "mod", "abs", "tril",
             "pow", "acos", "expm1", "sinh", "sinc", "neg", "lgamma", "gammaincc", "gammainc", "square", "divide", "gammaln",
             "atan", "gcd", "lcm", "cast", "greater_equal", "erf", "greater_than", "tanh", "transpose", "flatten", "multiply",
             "logical_not", "log", "log2", "log10", "trunc", "frac", "digamma", "renorm", "multigammaln", "nan_to_num",
             "index_add", "index_put", "ldexp", "i0", "polygamma", "copysign", "bitwise_left_shift", "bitwise_right_shift",
             "masked_fill", "masked_scatter", "hypot", "index_fill"]
    out = {}
    for n in names:
        fn = globals().get(n)
        for mod in (M, MP, L):
            fn = fn or getattr(mod, n, None)
        if fn is None and hasattr(torch, n):
            fn = (lambda t: lambda x, *a, name=None, **k: as_tensor(t(_p(x), *[_p(v) for v in a], **k)))(getattr(torch, n))
        if fn is not None:
            out[n + "_"] = _inplace(fn)
    return out


# ------------------------------------------------------------------ functions
def less(x, y, name=None):
    return as_tensor(torch.lt(_p(x), _p(y)))


def bitwise_invert(x, name=None):
    return as_tensor(torch.bitwise_not(_p(x)))


def floor_mod(x, y, name=None):
    return as_tensor(torch.remainder(_p(x), _p(y)))


mod = floor_mod


def block_diag(inputs, name=None):
    return as_tensor(torch.block_diag(*[_p(t) for t in inputs]))


def diag_embed(input, offset=0, dim1=-2, dim2=-1):
    return as_tensor(torch.diag_embed(_p(input), offset, dim1, dim2))


def cartesian_prod(x, name=None):
    return as_tensor(torch.cartesian_prod(*[_p(t) for t in x]))


def combinations(x, r=2, with_replacement=False, name=None):
    return as_tensor(torch.combinations(_p(x), r, with_replacement))


def slice_scatter(x, value, axes, starts, ends, strides, name=None):
    out = _p(x).clone()
    idx = [slice(None)] * out.dim()
    for a, s, e_, st in zip(axes, starts, ends, strides):
        idx[a] = slice(s, e_, st)
    out[tuple(idx)] = _p(value)
    return as_tensor(out)


def hsplit(x, num_or_indices, name=None):
    return [as_tensor(t) for t in torch.hsplit(_p(x), num_or_indices)]


def vsplit(x, num_or_indices, name=None):
    return [as_tensor(t) for t in torch.vsplit(_p(x), num_or_indices)]


def dsplit(x, num_or_indices, name=None):
    return [as_tensor(t) for t in torch.dsplit(_p(x), num_or_indices)]


def column_stack(x, name=None):
    return as_tensor(torch.column_stack([_p(t) for t in x]))


def row_stack(x, name=None):
    return as_tensor(torch.vstack([_p(t) for t in x]))


def reverse(x, axis, name=None):
    return as_tensor(torch.flip(_p(x), [axis] if isinstance(axis, int) else list(axis)))


def matrix_transpose(x, name=None):
    return as_tensor(_p(x).transpose(-1, -2))


def isin(x, test_x, assume_unique=False, invert=False, name=None):
    return as_tensor(torch.isin(_p(x), _p(test_x), assume_unique=assume_unique, invert=invert))


def isneginf(x, name=None):
    return as_tensor(torch.isneginf(_p(x)))


def isposinf(x, name=None):
    return as_tensor(torch.isposinf(_p(x)))


def histogram_bin_edges(input, bins=100, min=0, max=0, name=None):
    t = _p(input).float()
    lo, hi = (float(t.min()), float(t.max())) if min == 0 and max == 0 else (float(min), float(max))
    if lo == hi:
        lo, hi = lo - 0.5, hi + 0.5
    return as_tensor(torch.linspace(lo, hi, bins + 1))


def pdist(x, p=2.0, compute_mode="use_mm_for_euclid_dist_if_necessary", name=None):
    return as_tensor(torch.pdist(_p(x), p))


def nanquantile(x, q, axis=None, keepdim=False, interpolation="linear", name=None):
    t = _p(x)
    qq = torch.as_tensor(q, dtype=t.dtype if t.is_floating_point() else torch.float32)
    if axis is None:
        return as_tensor(torch.nanquantile(t.reshape(-1), qq, dim=0, keepdim=keepdim, interpolation=interpolation))
    return as_tensor(torch.nanquantile(t, qq, dim=axis, keepdim=keepdim, interpolation=interpolation))


def sinc(x, name=None):
    return as_tensor(torch.sinc(_p(x)))


def gammaln(x, name=None):
    return as_tensor(torch.lgamma(_p(x)))


def gammainc(x, y, name=None):
    return as_tensor(torch.special.gammainc(_p(x), _p(y)))


def gammaincc(x, y, name=None):
    return as_tensor(torch.special.gammaincc(_p(x), _p(y)))


def multigammaln(x, p, name=None):
    return as_tensor(torch.special.multigammaln(_p(x), p))


def polygamma(x, n, name=None):
    return as_tensor(torch.special.polygamma(n, _p(x)))


def i0e(x, name=None):
    return as_tensor(torch.special.i0e(_p(x)))


def i1(x, name=None):
    return as_tensor(torch.special.i1(_p(x)))


def i1e(x, name=None):
    return as_tensor(torch.special.i1e(_p(x)))


def vecdot(x, y, axis=-1, name=None):
    return as_tensor(torch.linalg.vecdot(_p(x), _p(y), dim=axis))


def reduce_as(x, target, name=None):
    """Sum ``x`` over the leading / broadcast dimensions so that the result has ``target``'s shape."""
    t = _p(x)
    ts = list(target.shape)
    while t.dim() > len(ts):
        t = t.sum(0)
    for d, (a, b) in enumerate(zip(t.shape, ts)):
        if a != b:
            t = t.sum(d, keepdim=True)
    return as_tensor(t)


def cumulative_trapezoid(y, x=None, dx=None, axis=-1, name=None):
    return as_tensor(torch.cumulative_trapezoid(_p(y), x=_p(x), dim=axis) if x is not None else
                     torch.cumulative_trapezoid(_p(y), dx=1.0 if dx is None else dx, dim=axis))


def unfold(x, axis, size, step, name=None):
    return as_tensor(_p(x).unfold(axis, size, step))


def log_normal(mean=1.0, std=2.0, shape=None, name=None):
    return as_tensor(torch.empty(list(shape or [1])).log_normal_(mean, std))


def log_normal_(x, mean=1.0, std=2.0, name=None):
    _p(x).log_normal_(mean, std)
    return x


def bernoulli_(x, p=0.5, name=None):
    _p(x).bernoulli_(p)
    return x


def cauchy_(x, loc=0, scale=1, name=None):
    _p(x).cauchy_(loc, scale)
    return x


def geometric_(x, probs, name=None):
    _p(x).geometric_(probs)
    return x


def from_dlpack(dlpack):
    return as_tensor(torch.utils.dlpack.from_dlpack(dlpack))


def to_dlpack(x):
    return torch.utils.dlpack.to_dlpack(_p(x))


def create_parameter(shape, dtype, name=None, attr=None, is_bias=False, default_initializer=None):
    from ..nn.layer.layers import Layer
    helper = Layer()
    return helper.create_parameter(list(shape), attr=attr, dtype=dtype, is_bias=is_bias, default_initializer=default_initializer)


def batch(reader, batch_size, drop_last=False):
    """Legacy reader decorator: groups the samples of ``reader()`` into lists of ``batch_size``."""
    def batched():
        buf = []
        for item in reader():
            buf.append(item)
            if len(buf) == batch_size:
                yield buf
                buf = []
        if buf and not drop_last:
            yield buf
    return batched


class iinfo:
    def __init__(self, dtype):
        i = torch.iinfo(_dt.to_torch(dtype))
        self.min, self.max, self.bits, self.dtype = i.min, i.max, i.bits, _dt.to_name(_dt.to_torch(dtype))

    def __repr__(self):
        return f"paddle.iinfo(min={self.min}, max={self.max}, bits={self.bits}, dtype={self.dtype})"


class finfo:
    def __init__(self, dtype):
        f = torch.finfo(_dt.to_torch(dtype))
        self.min, self.max, self.eps, self.tiny, self.resolution, self.bits = f.min, f.max, f.eps, f.tiny, f.resolution, f.bits
        self.smallest_normal, self.dtype = f.smallest_normal, _dt.to_name(_dt.to_torch(dtype))

    def __repr__(self):
        return (f"paddle.finfo(min={self.min}, max={self.max}, eps={self.eps}, resolution={self.resolution}, "
                f"smallest_normal={self.smallest_normal}, tiny={self.tiny}, bits={self.bits}, dtype={self.dtype})")


pstring, raw = "pstring", "raw"


def top_p_sampling(x, ps, threshold=None, topp_seed=None, seed=-1, k=0, mode="truncated", return_top=False, name=None):
    """Nucleus sampling over the last axis of probabilities ``x`` [batch, vocab] with per-row ``ps`` [batch, 1]:
    returns ``(sampled probability [batch, 1], sampled id [batch, 1])`` (python/paddle/tensor/search.py
    ``top_p_sampling``)."""
    import torch
    from .._core.tensor import as_tensor
    if (x.is_cuda and x.dim() == 2 and threshold is None and mode == "truncated" and not return_top
            and x.shape[1] * 4 <= 200 * 1024 and x.dtype in (torch.bfloat16, torch.float32)):
        # one kernel per call, no sort: bisection on the probability value inside shared memory
        from ..ops import functional as K
        from ..ops import native
        if K.get_kernel_policy() == "fused":
            xt = x.as_subclass(torch.Tensor)
            xt = xt if xt.stride(1) == 1 else xt.contiguous()
            if seed is not None and seed >= 0:
                sd, off = int(seed), 0
            else:
                gen = torch.cuda.default_generators[torch.cuda.current_device()]
                sd, off = gen.initial_seed(), gen.get_offset()
                gen.set_offset(off + 4)
            ids, probs = native.sample_top_p_top_k(xt, ps.as_subclass(torch.Tensor), k or 0, 1.0, sd, off, input_is_prob=True)
            return as_tensor(probs.to(x.dtype).reshape(-1, 1)), as_tensor(ids.reshape(-1, 1))
    p = x.as_subclass(torch.Tensor).float()
    tp = ps.as_subclass(torch.Tensor).float().reshape(-1, 1)
    sp, si = torch.sort(p, dim=-1, descending=True)
    cum = torch.cumsum(sp, -1)
    keep = (cum - sp) < tp                                   # the token that crosses the threshold stays in
    if k and k > 0:
        keep[:, k:] = False
    if threshold is not None:
        keep &= sp >= threshold.as_subclass(torch.Tensor).float().reshape(-1, 1)
    keep[:, 0] = True
    sp = torch.where(keep, sp, torch.zeros_like(sp))
    g = None
    if seed is not None and seed >= 0:
        g = torch.Generator(device=p.device)
        g.manual_seed(int(seed))
    pick = torch.multinomial(sp / sp.sum(-1, keepdim=True), 1, generator=g)
    ids = si.gather(-1, pick)
    probs = p.gather(-1, ids).to(x.dtype)
    return as_tensor(probs), as_tensor(ids)


def put_along_axis_(arr, indices, values, axis, reduce="assign", include_self=True, broadcast=True):
    import torch
    from .manipulation import put_along_axis
    out = put_along_axis(arr, indices, values, axis, reduce, include_self, broadcast)
    arr.as_subclass(torch.Tensor).copy_(out.as_subclass(torch.Tensor))
    return arr
