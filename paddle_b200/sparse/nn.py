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
