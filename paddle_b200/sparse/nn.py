"""``paddle.sparse.nn``: activations and layers acting on the stored values of sparse tensors."""
from __future__ import annotations

import torch

from ..nn.layer.layers import Layer


def _vals(fn, x):
    if x.layout == torch.sparse_csr:
        return torch.sparse_csr_tensor(x.crow_indices(), x.col_indices(), fn(x.values()), x.shape)
    x = x.coalesce()
    return torch.sparse_coo_tensor(x.indices(), fn(x.values()), x.shape)


class functional:
    @staticmethod
    def relu(x, name=None):
        return _vals(torch.relu, x)

    @staticmethod
    def relu6(x, name=None):
        return _vals(torch.nn.functional.relu6, x)

    @staticmethod
    def leaky_relu(x, negative_slope=0.01, name=None):
        return _vals(lambda v: torch.nn.functional.leaky_relu(v, negative_slope), x)

    @staticmethod
    def softmax(x, axis=-1, name=None):
        return torch.sparse.softmax(x.to_sparse_coo() if x.layout == torch.sparse_csr else x, dim=axis)

    @staticmethod
    def attention(query, key, value, sparse_mask, key_padding_mask=None, attn_mask=None, name=None):
        d = query.shape[-1]
        s = torch.matmul(query, key.transpose(-1, -2)) / (d ** 0.5)
        mask = sparse_mask.to_dense().reshape(s.shape) != 0
        s = s.masked_fill(~mask, float("-inf"))
        if attn_mask is not None:
            s = s + attn_mask
        return torch.matmul(torch.nan_to_num(torch.softmax(s, -1)), value)


class ReLU(Layer):
    def forward(self, x):
        return functional.relu(x)


class ReLU6(Layer):
    def forward(self, x):
        return functional.relu6(x)


class LeakyReLU(Layer):
    def __init__(self, negative_slope=0.01, name=None):
        super().__init__()
        self.negative_slope = negative_slope

    def forward(self, x):
        return functional.leaky_relu(x, self.negative_slope)


class Softmax(Layer):
    def __init__(self, axis=-1, name=None):
        super().__init__()
        self.axis = axis

    def forward(self, x):
        return functional.softmax(x, self.axis)


class BatchNorm(Layer):
    """Batch normalisation over the channel (last) dimension of the stored values."""

    def __init__(self, num_features, momentum=0.9, epsilon=1e-5, weight_attr=None, bias_attr=None, data_format="NDHWC",
                 use_global_stats=None, name=None):
        super().__init__()
        from .. import nn
        self.bn = nn.BatchNorm1D(num_features, momentum=momentum, epsilon=epsilon)

    def forward(self, x):
        return _vals(lambda v: self.bn(v), x)


# ----------------------------------------------------------------------------- convolution / pooling on COO tensors
# Layout: [N, D, H, W, C] (or [N, H, W, C]) with the channel dimension dense, as in python/paddle/sparse/nn/layer/conv.py.
# The arithmetic runs on the dense tensor cores (the active-site gather/scatter formulation only pays at very low
# density); what is sparse-specific is the OUTPUT pattern: a regular convolution activates every site its kernel
# touches, a submanifold convolution keeps exactly the input's active sites.
def _dense_channels_first(x, nd):
    d = x.to_dense()
    perm = [0, nd + 1] + list(range(1, nd + 1))
    return d.permute(perm)


def _to_sparse_channels_last(y, nd, sites=None):
    perm = [0] + list(range(2, nd + 2)) + [1]
    y = y.permute(perm).contiguous()
    if sites is None:
        active = (y != 0).any(-1)
    else:
        active = sites
    idx = active.nonzero().t().contiguous()
    vals = y[tuple(idx)]
    return torch.sparse_coo_tensor(idx, vals, y.shape)


def _active_sites(x, nd):
    x = x.coalesce()
    m = torch.zeros(x.shape[:nd + 1], dtype=torch.bool, device=x.values().device)
    m[tuple(x.indices()[:nd + 1])] = True
    return m


def _conv(x, weight, bias, stride, padding, dilation, groups, nd, subm):
    """``weight``: [*kernel, C_in / groups, C_out] (the reference's layout)."""
    xd = _dense_channels_first(x, nd)
    w = weight.as_subclass(torch.Tensor) if isinstance(weight, torch.Tensor) else weight
    perm = [nd + 1, nd] + list(range(nd))
    wt = w.permute(perm)
    fn = torch.nn.functional.conv3d if nd == 3 else torch.nn.functional.conv2d
    if subm:
        k = w.shape[:nd]
        dil = (dilation,) * nd if isinstance(dilation, int) else tuple(dilation)
        padding = [d_ * (kk - 1) // 2 for kk, d_ in zip(k, dil)]
        stride = 1
    b = bias.as_subclass(torch.Tensor) if isinstance(bias, torch.Tensor) else bias
    if subm:
        y = fn(xd, wt, None, stride, padding, dilation, groups)
        sites = _active_sites(x, nd)
        if b is not None:
            y = y + b.reshape(1, -1, *([1] * nd))
        return _to_sparse_channels_last(y, nd, sites)
    y = fn(xd, wt, None, stride, padding, dilation, groups)
    # a site is active if any input site falls under the kernel footprint
    ones = torch.ones((1, 1) + tuple(w.shape[:nd]), dtype=xd.dtype, device=xd.device)
    occ = fn(_active_sites(x, nd).to(xd.dtype).unsqueeze(1), ones, None, stride, padding, dilation) > 0
    if b is not None:
        y = y + b.reshape(1, -1, *([1] * nd))
    return _to_sparse_channels_last(y, nd, occ[:, 0])


def _f_conv3d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, data_format="NDHWC", name=None):
    return _conv(x, weight, bias, stride, padding, dilation, groups, 3, False)


def _f_subm_conv3d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, data_format="NDHWC", key=None, name=None):
    return _conv(x, weight, bias, stride, padding, dilation, groups, 3, True)


def _f_conv2d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, data_format="NHWC", name=None):
    return _conv(x, weight, bias, stride, padding, dilation, groups, 2, False)


def _f_subm_conv2d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, data_format="NHWC", key=None, name=None):
    return _conv(x, weight, bias, stride, padding, dilation, groups, 2, True)


def _f_max_pool3d(x, kernel_size, stride=None, padding=0, ceil_mode=False, data_format="NDHWC", name=None):
    xd = _dense_channels_first(x, 3)
    sites = _active_sites(x, 3).to(xd.dtype).unsqueeze(1)
    neg = torch.where(sites.expand_as(xd) > 0, xd, torch.full_like(xd, float("-inf")))
    y = torch.nn.functional.max_pool3d(neg, kernel_size, stride, padding, ceil_mode=ceil_mode)
    occ = torch.nn.functional.max_pool3d(sites, kernel_size, stride, padding, ceil_mode=ceil_mode) > 0
    y = torch.where(torch.isinf(y), torch.zeros_like(y), y)
    return _to_sparse_channels_last(y, 3, occ[:, 0])


for _n, _f in (("conv3d", _f_conv3d), ("subm_conv3d", _f_subm_conv3d), ("conv2d", _f_conv2d), ("subm_conv2d", _f_subm_conv2d),
               ("subm_conv3d_igemm", _f_subm_conv3d), ("subm_conv2d_igemm", _f_subm_conv2d), ("max_pool3d", _f_max_pool3d)):
    setattr(functional, _n, staticmethod(_f))


class _SparseConv(Layer):
    _nd, _subm = 3, False

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 padding_mode="zeros", key=None, weight_attr=None, bias_attr=None, data_format=None):
        super().__init__()
        k = (kernel_size,) * self._nd if isinstance(kernel_size, int) else tuple(kernel_size)
        self._stride, self._padding, self._dilation, self._groups = stride, padding, dilation, groups
        self.weight = self.create_parameter([*k, in_channels // groups, out_channels], attr=weight_attr)
        self.bias = None if bias_attr is False else self.create_parameter([out_channels], attr=bias_attr, is_bias=True)

    def forward(self, x):
        return _conv(x, self.weight, self.bias, self._stride, self._padding, self._dilation, self._groups, self._nd,
                     self._subm)


class Conv3D(_SparseConv):
    pass


class SubmConv3D(_SparseConv):
    _subm = True


class Conv2D(_SparseConv):
    _nd = 2


class SubmConv2D(_SparseConv):
    _nd, _subm = 2, True


class MaxPool3D(Layer):
    def __init__(self, kernel_size, stride=None, padding=0, return_mask=False, ceil_mode=False, data_format="NDHWC",
                 name=None):
        super().__init__()
        self._k, self._s, self._p, self._c = kernel_size, stride, padding, ceil_mode

    def forward(self, x):
        return _f_max_pool3d(x, self._k, self._s, self._p, self._c)


class SyncBatchNorm(BatchNorm):
    """Batch statistics all-reduced over the data-parallel group (values of active sites only)."""

    def forward(self, x):
        import torch.distributed as tdist
        if not (self.training and tdist.is_available() and tdist.is_initialized() and tdist.get_world_size() > 1):
            return super().forward(x)
        xc = x.coalesce()
        v = xc.values()
        stats = torch.cat([v.sum(0), (v * v).sum(0), torch.tensor([float(v.shape[0])], device=v.device, dtype=v.dtype)])
        tdist.all_reduce(stats)
        c = v.shape[1]
        n = stats[-1]
        mean, var = stats[:c] / n, stats[c:2 * c] / n - (stats[:c] / n) ** 2
        bn = self.bn
        with torch.no_grad():
            m = 1.0 - bn._momentum if hasattr(bn, "_momentum") else 0.1
            bn._mean.as_subclass(torch.Tensor).mul_(1 - m).add_(mean.detach(), alpha=m)
            bn._variance.as_subclass(torch.Tensor).mul_(1 - m).add_(var.detach() * n / (n - 1).clamp_min(1), alpha=m)
        out = (v - mean) / torch.sqrt(var + bn._eps)
        if bn.weight is not None:
            out = out * bn.weight.as_subclass(torch.Tensor) + bn.bias.as_subclass(torch.Tensor)
        return torch.sparse_coo_tensor(xc.indices(), out, xc.shape)

    @classmethod
    def convert_sync_batchnorm(cls, layer):
        return layer


import sys as _sys  # noqa: E402
import types as _types  # noqa: E402


def _namespace_module(ns, name):
    m = _types.ModuleType(name)
    from .tensor import api
    for k, v in vars(ns).items():
        if not k.startswith("__"):
            f = v.__func__ if isinstance(v, staticmethod) else v
            setattr(m, k, api(f) if callable(f) else f)       # take and return SparseTensor
    _sys.modules[name] = m
    return m


functional = _namespace_module(functional, __name__ + ".functional")


# layers take and return SparseTensor
from .tensor import api as _api  # noqa: E402
for _cls in (ReLU, ReLU6, LeakyReLU, Softmax, BatchNorm, SyncBatchNorm, Conv3D, SubmConv3D, Conv2D, SubmConv2D, MaxPool3D):
    if "forward" in vars(_cls):
        _cls.forward = _api(_cls.forward)
_SparseConv.forward = _api(_SparseConv.forward)
del _cls
