"""Layer classes of ``paddle.nn`` (python/paddle/nn/layer/{common,activation,norm,conv,pooling,loss,
container,transformer,rnn}.py in the reference), built on :class:`Layer` and ``nn.functional``."""
from __future__ import annotations

import collections
import math

import numpy as np
import torch

from ..._core import dtype as _dt
from ..._core.tensor import EagerParamBase, as_tensor
from .. import functional as F
from ..initializer import Constant, KaimingUniform, Normal, Uniform, XavierUniform
from .layers import Layer, ParamAttr


# ------------------------------------------------------------------ containers
class Sequential(Layer):
    def __init__(self, *layers):
        super().__init__()
        if len(layers) == 1 and isinstance(layers[0], (list, tuple)) and layers[0] and isinstance(layers[0][0], (list, tuple)):
            layers = layers[0]
        for i, l in enumerate(layers):
            if isinstance(l, (list, tuple)):
                self.add_sublayer(l[0], l[1])
            else:
                self.add_sublayer(str(i), l)

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return Sequential(*list(self._sub_layers.values())[idx])
        if isinstance(idx, str):
            return self._sub_layers[idx]
        return list(self._sub_layers.values())[idx]

    def __len__(self):
        return len(self._sub_layers)

    def __iter__(self):
        return iter(self._sub_layers.values())

    def append(self, layer):
        self.add_sublayer(str(len(self._sub_layers)), layer)

    def forward(self, x):
        for l in self._sub_layers.values():
            x = l(x)
        return x


class LayerList(Layer):
    def __init__(self, sublayers=None):
        super().__init__()
        if sublayers is not None:
            for i, l in enumerate(sublayers):
                self.add_sublayer(str(i), l)

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return LayerList(list(self._sub_layers.values())[idx])
        n = len(self._sub_layers)
        return self._sub_layers[str(idx if idx >= 0 else idx + n)]

    def __setitem__(self, idx, layer):
        self._sub_layers[str(idx)] = layer

    def __len__(self):
        return len(self._sub_layers)

    def __iter__(self):
        return iter(self._sub_layers.values())

    def append(self, layer):
        self.add_sublayer(str(len(self._sub_layers)), layer)
        return self

    def extend(self, layers):
        for l in layers:
            self.append(l)
        return self

    def insert(self, index, layer):
        ls = list(self._sub_layers.values())
        ls.insert(index, layer)
        self._sub_layers.clear()
        for i, l in enumerate(ls):
            self._sub_layers[str(i)] = l


class LayerDict(Layer):
    def __init__(self, sublayers=None):
        super().__init__()
        if sublayers:
            self.update(sublayers)

    def __getitem__(self, k):
        return self._sub_layers[k]

    def __setitem__(self, k, v):
        self.add_sublayer(k, v)

    def __delitem__(self, k):
        del self._sub_layers[k]

    def __len__(self):
        return len(self._sub_layers)

    def __iter__(self):
        return iter(self._sub_layers)

    def __contains__(self, k):
        return k in self._sub_layers

    def keys(self):
        return self._sub_layers.keys()

    def values(self):
        return self._sub_layers.values()

    def items(self):
        return self._sub_layers.items()

    def update(self, sublayers):
        items = sublayers.items() if isinstance(sublayers, (dict, LayerDict)) else sublayers
        for k, v in items:
            self.add_sublayer(k, v)


class ParameterList(Layer):
    def __init__(self, parameters=None):
        super().__init__()
        if parameters is not None:
            for i, p in enumerate(parameters):
                self.add_parameter(str(i), p)

    def __getitem__(self, idx):
        return self._parameters[str(idx if idx >= 0 else idx + len(self._parameters))]

    def __len__(self):
        return len(self._parameters)

    def __iter__(self):
        return iter(self._parameters.values())

    def append(self, p):
        self.add_parameter(str(len(self._parameters)), p)
        return self


# ------------------------------------------------------------------ core layers
class Linear(Layer):
    """Weight is ``[in_features, out_features]`` (python/paddle/nn/layer/common.py ``Linear``)."""

    def __init__(self, in_features, out_features, weight_attr=None, bias_attr=None, name=None):
        super().__init__()
        self._in, self._out = in_features, out_features
        self.weight = self.create_parameter([in_features, out_features], weight_attr)
        self.bias = self.create_parameter([out_features], bias_attr, is_bias=True)

    def forward(self, x):
        return F.linear(x, self.weight, self.bias)

    def extra_repr(self):
        return f"in_features={self._in}, out_features={self._out}"


class Embedding(Layer):
    def __init__(self, num_embeddings, embedding_dim, padding_idx=None, sparse=False, weight_attr=None, name=None):
        super().__init__()
        self._padding_idx = padding_idx if padding_idx is None or padding_idx >= 0 else num_embeddings + padding_idx
        self.weight = self.create_parameter([num_embeddings, embedding_dim], weight_attr,
                                            default_initializer=Normal(0.0, 1.0))
        if self._padding_idx is not None:
            with torch.no_grad():
                self.weight[self._padding_idx].zero_()

    def forward(self, x):
        return F.embedding(x, self.weight, self._padding_idx)


class Identity(Layer):
    def __init__(self, *a, **k):
        super().__init__()

    def forward(self, x):
        return x


class Flatten(Layer):
    def __init__(self, start_axis=1, stop_axis=-1):
        super().__init__()
        self.start_axis, self.stop_axis = start_axis, stop_axis

    def forward(self, x):
        return torch.flatten(x, self.start_axis, self.stop_axis)


class Unflatten(Layer):
    def __init__(self, axis, shape, name=None):
        super().__init__()
        self.axis, self.shape = axis, tuple(shape)

    def forward(self, x):
        return torch.unflatten(x, self.axis, self.shape)


class Dropout(Layer):
    def __init__(self, p=0.5, axis=None, mode="upscale_in_train", name=None):
        super().__init__()
        self.p, self.axis, self.mode = p, axis, mode

    def forward(self, x):
        return F.dropout(x, self.p, self.axis, self.training, self.mode)


class Dropout2D(Layer):
    def __init__(self, p=0.5, data_format="NCHW", name=None):
        super().__init__()
        self.p = p

    def forward(self, x):
        return F.dropout2d(x, self.p, self.training)


class Dropout3D(Dropout2D):
    def forward(self, x):
        return F.dropout3d(x, self.p, self.training)


class AlphaDropout(Dropout2D):
    def forward(self, x):
        return F.alpha_dropout(x, self.p, self.training)


class LayerNorm(Layer):
    def __init__(self, normalized_shape, epsilon=1e-5, weight_attr=None, bias_attr=None, name=None):
        super().__init__()
        self._shape = [normalized_shape] if isinstance(normalized_shape, int) else list(normalized_shape)
        self._eps = epsilon
        self.weight = self.create_parameter(self._shape, weight_attr, default_initializer=Constant(1.0)) \
            if weight_attr is not False else None
        self.bias = self.create_parameter(self._shape, bias_attr, is_bias=True) if bias_attr is not False else None

    def forward(self, x):
        return F.layer_norm(x, self._shape, self.weight, self.bias, self._eps)


class RMSNorm(Layer):
    def __init__(self, hidden_size, epsilon=1e-6, weight_attr=None, name=None):
        super().__init__()
        self._eps = epsilon
        self.weight = self.create_parameter([hidden_size], weight_attr, default_initializer=Constant(1.0))

    def forward(self, x):
        return F.rms_norm(x, self.weight, self._eps)


class _BatchNormBase(Layer):
    def __init__(self, num_features, momentum=0.9, epsilon=1e-5, weight_attr=None, bias_attr=None,
                 data_format="NCHW", use_global_stats=None, name=None):
        super().__init__()
        self._momentum, self._eps, self._fmt, self._ugs = momentum, epsilon, data_format, use_global_stats
        self.weight = self.create_parameter([num_features], weight_attr, default_initializer=Constant(1.0)) \
            if weight_attr is not False else None
        self.bias = self.create_parameter([num_features], bias_attr, is_bias=True) if bias_attr is not False else None
        self.register_buffer("_mean", torch.zeros(num_features, device=_dt.default_device()))
        self.register_buffer("_variance", torch.ones(num_features, device=_dt.default_device()))

    def forward(self, x):
        return F.batch_norm(x, self._mean, self._variance, self.weight, self.bias, self.training, self._momentum,
                            self._eps, self._fmt, self._ugs)


class BatchNorm1D(_BatchNormBase):
    def __init__(self, num_features, momentum=0.9, epsilon=1e-5, weight_attr=None, bias_attr=None,
                 data_format="NCL", use_global_stats=None, name=None):
        super().__init__(num_features, momentum, epsilon, weight_attr, bias_attr, data_format, use_global_stats)


class BatchNorm2D(_BatchNormBase):
    pass


class BatchNorm3D(_BatchNormBase):
    def __init__(self, num_features, momentum=0.9, epsilon=1e-5, weight_attr=None, bias_attr=None,
                 data_format="NCDHW", use_global_stats=None, name=None):
        super().__init__(num_features, momentum, epsilon, weight_attr, bias_attr, data_format, use_global_stats)


class BatchNorm(_BatchNormBase):
    def __init__(self, num_channels, act=None, is_test=False, momentum=0.9, epsilon=1e-5, param_attr=None,
                 bias_attr=None, dtype="float32", data_layout="NCHW", **kw):
        super().__init__(num_channels, momentum, epsilon, param_attr, bias_attr, data_layout)
        self._act = act

    def forward(self, x):
        y = super().forward(x)
        return getattr(F, self._act)(y) if self._act else y


class SyncBatchNorm(_BatchNormBase):
    """Batch norm whose statistics are all-reduced over the data-parallel group in training."""

    def forward(self, x):
        from ...distributed import collective as C
        if not self.training or not C.is_initialized() or C.get_world_size() == 1:
            return super().forward(x)
        dims = [0] + list(range(2, x.dim()))
        n = torch.tensor([x.numel() / x.shape[1]], device=x.device, dtype=torch.float32)
        s = x.float().sum(dims)
        ss = (x.float() ** 2).sum(dims)
        packed = torch.cat([s, ss, n])
        C.all_reduce(packed)
        C_ = x.shape[1]
        tot = packed[-1]
        mean = packed[:C_] / tot
        var = packed[C_:2 * C_] / tot - mean ** 2
        with torch.no_grad():
            self._mean.mul_(self._momentum).add_(mean.detach() * (1 - self._momentum))
            self._variance.mul_(self._momentum).add_(var.detach() * (1 - self._momentum))
        shape = [1, C_] + [1] * (x.dim() - 2)
        y = (x - mean.view(shape).to(x.dtype)) * torch.rsqrt(var.view(shape) + self._eps).to(x.dtype)
        if self.weight is not None:
            y = y * self.weight.view(shape) + self.bias.view(shape)
        return y

    @classmethod
    def convert_sync_batchnorm(cls, layer):
        for name, sub in list(layer._sub_layers.items()):
            if isinstance(sub, _BatchNormBase) and not isinstance(sub, SyncBatchNorm):
                new = cls(sub.weight.shape[0], sub._momentum, sub._eps)
                new.weight, new.bias = sub.weight, sub.bias
                new._buffers["_mean"], new._buffers["_variance"] = sub._mean, sub._variance
                layer._sub_layers[name] = new
            else:
                cls.convert_sync_batchnorm(sub)
        return layer


class GroupNorm(Layer):
    def __init__(self, num_groups, num_channels, epsilon=1e-5, weight_attr=None, bias_attr=None, data_format="NCHW",
                 name=None):
        super().__init__()
        self._g, self._eps, self._fmt = num_groups, epsilon, data_format
        self.weight = self.create_parameter([num_channels], weight_attr, default_initializer=Constant(1.0))
        self.bias = self.create_parameter([num_channels], bias_attr, is_bias=True)

    def forward(self, x):
        return F.group_norm(x, self._g, self._eps, self.weight, self.bias, self._fmt)


class InstanceNorm2D(Layer):
    def __init__(self, num_features, epsilon=1e-5, momentum=0.9, weight_attr=None, bias_attr=None,
                 data_format="NCHW", name=None):
        super().__init__()
        self._eps = epsilon
        self.scale = self.create_parameter([num_features], weight_attr, default_initializer=Constant(1.0)) \
            if weight_attr is not False else None
        self.bias = self.create_parameter([num_features], bias_attr, is_bias=True) if bias_attr is not False else None

    def forward(self, x):
        return F.instance_norm(x, weight=self.scale, bias=self.bias, eps=self._eps)


InstanceNorm1D = InstanceNorm3D = InstanceNorm2D


class LocalResponseNorm(Layer):
    def __init__(self, size, alpha=1e-4, beta=0.75, k=1.0, data_format="NCHW", name=None):
        super().__init__()
        self.a = (size, alpha, beta, k)

    def forward(self, x):
        return F.local_response_norm(x, *self.a)


# ------------------------------------------------------------------ activations as layers
def _act_layer(name, fn, *defaults):
    def __init__(self, *args, **kw):
        Layer.__init__(self)
        kw.pop("name", None)
        self._args, self._kw = args, kw

    def forward(self, x):
        return fn(x, *self._args, **self._kw)

    return type(name, (Layer,), {"__init__": __init__, "forward": forward})


ReLU = _act_layer("ReLU", F.relu)
ReLU6 = _act_layer("ReLU6", F.relu6)
GELU = _act_layer("GELU", F.gelu)
Silu = _act_layer("Silu", F.silu)
Swish = _act_layer("Swish", F.silu)
Sigmoid = _act_layer("Sigmoid", F.sigmoid)
Tanh = _act_layer("Tanh", F.tanh)
LeakyReLU = _act_layer("LeakyReLU", F.leaky_relu)
ELU = _act_layer("ELU", F.elu)
SELU = _act_layer("SELU", F.selu)
CELU = _act_layer("CELU", F.celu)
Hardtanh = _act_layer("Hardtanh", F.hardtanh)
Hardsigmoid = _act_layer("Hardsigmoid", F.hardsigmoid)
Hardswish = _act_layer("Hardswish", F.hardswish)
Hardshrink = _act_layer("Hardshrink", F.hardshrink)
Softshrink = _act_layer("Softshrink", F.softshrink)
Tanhshrink = _act_layer("Tanhshrink", F.tanhshrink)
ThresholdedReLU = _act_layer("ThresholdedReLU", F.thresholded_relu)
Softplus = _act_layer("Softplus", F.softplus)
Softsign = _act_layer("Softsign", F.softsign)
Mish = _act_layer("Mish", F.mish)
LogSigmoid = _act_layer("LogSigmoid", F.log_sigmoid)
Softmax = _act_layer("Softmax", F.softmax)
LogSoftmax = _act_layer("LogSoftmax", F.log_softmax)
GLU = _act_layer("GLU", F.glu)
Maxout = _act_layer("Maxout", F.maxout)
RReLU = _act_layer("RReLU", F.rrelu)


class PReLU(Layer):
    def __init__(self, num_parameters=1, init=0.25, weight_attr=None, data_format="NCHW", name=None):
        super().__init__()
        self._weight = self.create_parameter([num_parameters], weight_attr, default_initializer=Constant(init))

    def forward(self, x):
        return F.prelu(x, self._weight)


# ------------------------------------------------------------------ conv / pool
class _ConvNd(Layer):
    _fn = None
    _nd = 2
    _transposed = False

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 padding_mode="zeros", weight_attr=None, bias_attr=None, data_format=None, output_padding=0, name=None):
        super().__init__()
        ks = tuple(kernel_size) if isinstance(kernel_size, (list, tuple)) else (kernel_size,) * self._nd
        self._stride, self._padding, self._dilation, self._groups = stride, padding, dilation, groups
        self._output_padding = output_padding
        self._data_format = data_format
        if self._transposed:
            shape = [in_channels, out_channels // groups, *ks]
        else:
            shape = [out_channels, in_channels // groups, *ks]
        fan_in = (in_channels // groups) * int(np.prod(ks))
        self.weight = self.create_parameter(shape, weight_attr, default_initializer=Normal(0.0, math.sqrt(2.0 / fan_in)))
        self.bias = self.create_parameter([out_channels], bias_attr, is_bias=True)

    def forward(self, x):
        kw = {}
        if self._data_format:
            kw["data_format"] = self._data_format
        if self._transposed:
            return type(self)._fn(x, self.weight, self.bias, self._stride, self._padding, self._output_padding,
                                  groups=self._groups, dilation=self._dilation, **kw)
        return type(self)._fn(x, self.weight, self.bias, self._stride, self._padding, self._dilation, self._groups, **kw)


class Conv1D(_ConvNd):
    _fn, _nd = staticmethod(F.conv1d), 1


class Conv2D(_ConvNd):
    _fn, _nd = staticmethod(F.conv2d), 2


class Conv3D(_ConvNd):
    _fn, _nd = staticmethod(F.conv3d), 3


class Conv1DTranspose(_ConvNd):
    _fn, _nd, _transposed = staticmethod(F.conv1d_transpose), 1, True


class Conv2DTranspose(_ConvNd):
    _fn, _nd, _transposed = staticmethod(F.conv2d_transpose), 2, True


class Conv3DTranspose(_ConvNd):
    _fn, _nd, _transposed = staticmethod(F.conv3d_transpose), 3, True


def _pool_layer(name, fn):
    def __init__(self, kernel_size=None, stride=None, padding=0, **kw):
        Layer.__init__(self)
        kw.pop("name", None)
        self._a = (kernel_size, stride, padding)
        self._kw = kw

    def forward(self, x):
        return fn(x, *self._a, **self._kw)

    return type(name, (Layer,), {"__init__": __init__, "forward": forward})


MaxPool1D = _pool_layer("MaxPool1D", F.max_pool1d)
MaxPool2D = _pool_layer("MaxPool2D", F.max_pool2d)
MaxPool3D = _pool_layer("MaxPool3D", F.max_pool3d)
AvgPool1D = _pool_layer("AvgPool1D", F.avg_pool1d)
AvgPool2D = _pool_layer("AvgPool2D", F.avg_pool2d)
AvgPool3D = _pool_layer("AvgPool3D", F.avg_pool3d)


def _adaptive_layer(name, fn):
    def __init__(self, output_size, **kw):
        Layer.__init__(self)
        kw.pop("name", None)
        kw.pop("data_format", None)
        self._o, self._kw = output_size, kw

    def forward(self, x):
        return fn(x, self._o, **self._kw)

    return type(name, (Layer,), {"__init__": __init__, "forward": forward})


AdaptiveAvgPool1D = _adaptive_layer("AdaptiveAvgPool1D", F.adaptive_avg_pool1d)
AdaptiveAvgPool2D = _adaptive_layer("AdaptiveAvgPool2D", F.adaptive_avg_pool2d)
AdaptiveAvgPool3D = _adaptive_layer("AdaptiveAvgPool3D", F.adaptive_avg_pool3d)
AdaptiveMaxPool1D = _adaptive_layer("AdaptiveMaxPool1D", F.adaptive_max_pool1d)
AdaptiveMaxPool2D = _adaptive_layer("AdaptiveMaxPool2D", F.adaptive_max_pool2d)


class Upsample(Layer):
    def __init__(self, size=None, scale_factor=None, mode="nearest", align_corners=False, align_mode=0,
                 data_format="NCHW", name=None):
        super().__init__()
        self._a = dict(size=size, scale_factor=scale_factor, mode=mode, align_corners=align_corners,
                       data_format=data_format)

    def forward(self, x):
        return F.interpolate(x, **self._a)


class UpsamplingNearest2D(Upsample):
    def __init__(self, size=None, scale_factor=None, data_format="NCHW", name=None):
        super().__init__(size, scale_factor, "nearest", data_format=data_format)


class UpsamplingBilinear2D(Upsample):
    def __init__(self, size=None, scale_factor=None, data_format="NCHW", name=None):
        super().__init__(size, scale_factor, "bilinear", True, data_format=data_format)


class Pad1D(Layer):
    def __init__(self, padding, mode="constant", value=0.0, data_format="NCL", name=None):
        super().__init__()
        self._p = [padding] * 2 if isinstance(padding, int) else list(padding)
        self._mode, self._value, self._fmt = mode, value, data_format

    def forward(self, x):
        return F.pad(x, self._p, self._mode, self._value, self._fmt)


class Pad2D(Pad1D):
    def __init__(self, padding, mode="constant", value=0.0, data_format="NCHW", name=None):
        Layer.__init__(self)
        self._p = [padding] * 4 if isinstance(padding, int) else list(padding)
        self._mode, self._value, self._fmt = mode, value, data_format


class Pad3D(Pad1D):
    def __init__(self, padding, mode="constant", value=0.0, data_format="NCDHW", name=None):
        Layer.__init__(self)
        self._p = [padding] * 6 if isinstance(padding, int) else list(padding)
        self._mode, self._value, self._fmt = mode, value, data_format


ZeroPad2D = Pad2D


class PixelShuffle(Layer):
    def __init__(self, upscale_factor, data_format="NCHW", name=None):
        super().__init__()
        self._f = upscale_factor

    def forward(self, x):
        return F.pixel_shuffle(x, self._f)


class CosineSimilarity(Layer):
    def __init__(self, axis=1, eps=1e-8):
        super().__init__()
        self._axis, self._eps = axis, eps

    def forward(self, x1, x2):
        return F.cosine_similarity(x1, x2, self._axis, self._eps)


# ------------------------------------------------------------------ loss layers
def _loss_layer(name, fn, n_in=2):
    def __init__(self, *args, **kw):
        Layer.__init__(self)
        kw.pop("name", None)
        self._args, self._kw = args, kw

    def forward(self, *inputs):
        return fn(*inputs, *self._args, **self._kw)

    return type(name, (Layer,), {"__init__": __init__, "forward": forward})


class CrossEntropyLoss(Layer):
    def __init__(self, weight=None, ignore_index=-100, reduction="mean", soft_label=False, axis=-1, use_softmax=True,
                 label_smoothing=0.0, name=None):
        super().__init__()
        self._kw = dict(weight=weight, ignore_index=ignore_index, reduction=reduction, soft_label=soft_label,
                        axis=axis, use_softmax=use_softmax, label_smoothing=label_smoothing)

    def forward(self, input, label):
        return F.cross_entropy(input, label, **self._kw)


MSELoss = _loss_layer("MSELoss", F.mse_loss)
L1Loss = _loss_layer("L1Loss", F.l1_loss)
SmoothL1Loss = _loss_layer("SmoothL1Loss", F.smooth_l1_loss)
NLLLoss = _loss_layer("NLLLoss", F.nll_loss)
BCELoss = _loss_layer("BCELoss", F.binary_cross_entropy)
BCEWithLogitsLoss = _loss_layer("BCEWithLogitsLoss", F.binary_cross_entropy_with_logits)
KLDivLoss = _loss_layer("KLDivLoss", F.kl_div)
MarginRankingLoss = _loss_layer("MarginRankingLoss", F.margin_ranking_loss)
HingeEmbeddingLoss = _loss_layer("HingeEmbeddingLoss", F.hinge_embedding_loss)
CosineEmbeddingLoss = _loss_layer("CosineEmbeddingLoss", F.cosine_embedding_loss)
TripletMarginLoss = _loss_layer("TripletMarginLoss", F.triplet_margin_loss)
CTCLoss = _loss_layer("CTCLoss", F.ctc_loss)


# ------------------------------------------------------------------ transformer
class MultiHeadAttention(Layer):
    """python/paddle/nn/layer/transformer.py ``MultiHeadAttention`` (batch-first ``[b, s, e]``)."""

    def __init__(self, embed_dim, num_heads, dropout=0.0, kdim=None, vdim=None, need_weights=False,
                 weight_attr=None, bias_attr=None):
        super().__init__()
        self.embed_dim, self.num_heads, self.dropout = embed_dim, num_heads, dropout
        self.head_dim = embed_dim // num_heads
        self.need_weights = need_weights
        self.q_proj = Linear(embed_dim, embed_dim, weight_attr, bias_attr)
        self.k_proj = Linear(kdim or embed_dim, embed_dim, weight_attr, bias_attr)
        self.v_proj = Linear(vdim or embed_dim, embed_dim, weight_attr, bias_attr)
        self.out_proj = Linear(embed_dim, embed_dim, weight_attr, bias_attr)

    def forward(self, query, key=None, value=None, attn_mask=None, cache=None):
        key = query if key is None else key
        value = key if value is None else value
        b, sq = query.shape[0], query.shape[1]
        q = self.q_proj(query).reshape([b, sq, self.num_heads, self.head_dim])
        k = self.k_proj(key).reshape([b, key.shape[1], self.num_heads, self.head_dim])
        v = self.v_proj(value).reshape([b, value.shape[1], self.num_heads, self.head_dim])
        if attn_mask is not None and attn_mask.dtype == torch.bool:
            attn_mask = torch.zeros(attn_mask.shape, dtype=q.dtype, device=q.device).masked_fill(~attn_mask, float("-inf"))
        o = F.scaled_dot_product_attention(q, k, v, attn_mask, self.dropout, False, self.training)
        return self.out_proj(o.reshape([b, sq, self.embed_dim]))


class TransformerEncoderLayer(Layer):
    def __init__(self, d_model, nhead, dim_feedforward, dropout=0.1, activation="relu", attn_dropout=None,
                 act_dropout=None, normalize_before=False, weight_attr=None, bias_attr=None, layer_norm_eps=1e-5):
        super().__init__()
        self.normalize_before = normalize_before
        self.self_attn = MultiHeadAttention(d_model, nhead, attn_dropout if attn_dropout is not None else dropout,
                                            weight_attr=weight_attr, bias_attr=bias_attr)
        self.linear1 = Linear(d_model, dim_feedforward, weight_attr, bias_attr)
        self.linear2 = Linear(dim_feedforward, d_model, weight_attr, bias_attr)
        self.norm1 = LayerNorm(d_model, layer_norm_eps)
        self.norm2 = LayerNorm(d_model, layer_norm_eps)
        self.dropout = Dropout(act_dropout if act_dropout is not None else dropout)
        self.dropout1, self.dropout2 = Dropout(dropout), Dropout(dropout)
        self.activation = getattr(F, activation)

    def forward(self, src, src_mask=None, cache=None):
        r = src
        if self.normalize_before:
            src = self.norm1(src)
        src = r + self.dropout1(self.self_attn(src, src, src, src_mask))
        if not self.normalize_before:
            src = self.norm1(src)
        r = src
        if self.normalize_before:
            src = self.norm2(src)
        src = r + self.dropout2(self.linear2(self.dropout(self.activation(self.linear1(src)))))
        if not self.normalize_before:
            src = self.norm2(src)
        return src


class TransformerEncoder(Layer):
    def __init__(self, encoder_layer, num_layers, norm=None):
        super().__init__()
        import copy
        self.layers = LayerList([encoder_layer if i == 0 else copy.deepcopy(encoder_layer) for i in range(num_layers)])
        self.norm = norm

    def forward(self, src, src_mask=None, cache=None):
        for l in self.layers:
            src = l(src, src_mask)
        return self.norm(src) if self.norm is not None else src


class TransformerDecoderLayer(Layer):
    def __init__(self, d_model, nhead, dim_feedforward, dropout=0.1, activation="relu", attn_dropout=None,
                 act_dropout=None, normalize_before=False, weight_attr=None, bias_attr=None, layer_norm_eps=1e-5):
        super().__init__()
        self.normalize_before = normalize_before
        ad = attn_dropout if attn_dropout is not None else dropout
        self.self_attn = MultiHeadAttention(d_model, nhead, ad)
        self.cross_attn = MultiHeadAttention(d_model, nhead, ad)
        self.linear1, self.linear2 = Linear(d_model, dim_feedforward), Linear(dim_feedforward, d_model)
        self.norm1, self.norm2, self.norm3 = (LayerNorm(d_model, layer_norm_eps) for _ in range(3))
        self.dropout = Dropout(act_dropout if act_dropout is not None else dropout)
        self.dropout1, self.dropout2, self.dropout3 = Dropout(dropout), Dropout(dropout), Dropout(dropout)
        self.activation = getattr(F, activation)

    def forward(self, tgt, memory, tgt_mask=None, memory_mask=None, cache=None):
        def block(x, norm, fn, drop):
            r = x
            if self.normalize_before:
                x = norm(x)
            x = r + drop(fn(x))
            return x if self.normalize_before else norm(x)
        tgt = block(tgt, self.norm1, lambda t: self.self_attn(t, t, t, tgt_mask), self.dropout1)
        tgt = block(tgt, self.norm2, lambda t: self.cross_attn(t, memory, memory, memory_mask), self.dropout2)
        return block(tgt, self.norm3, lambda t: self.linear2(self.dropout(self.activation(self.linear1(t)))), self.dropout3)


class TransformerDecoder(Layer):
    def __init__(self, decoder_layer, num_layers, norm=None):
        super().__init__()
        import copy
        self.layers = LayerList([decoder_layer if i == 0 else copy.deepcopy(decoder_layer) for i in range(num_layers)])
        self.norm = norm

    def forward(self, tgt, memory, tgt_mask=None, memory_mask=None, cache=None):
        for l in self.layers:
            tgt = l(tgt, memory, tgt_mask, memory_mask)
        return self.norm(tgt) if self.norm is not None else tgt


class Transformer(Layer):
    def __init__(self, d_model=512, nhead=8, num_encoder_layers=6, num_decoder_layers=6, dim_feedforward=2048,
                 dropout=0.1, activation="relu", normalize_before=False, **kw):
        super().__init__()
        self.encoder = TransformerEncoder(TransformerEncoderLayer(d_model, nhead, dim_feedforward, dropout, activation,
                                                                  normalize_before=normalize_before),
                                          num_encoder_layers, LayerNorm(d_model) if normalize_before else None)
        self.decoder = TransformerDecoder(TransformerDecoderLayer(d_model, nhead, dim_feedforward, dropout, activation,
                                                                  normalize_before=normalize_before),
                                          num_decoder_layers, LayerNorm(d_model) if normalize_before else None)

    def forward(self, src, tgt, src_mask=None, tgt_mask=None, memory_mask=None):
        memory = self.encoder(src, src_mask)
        return self.decoder(tgt, memory, tgt_mask, memory_mask)

    @staticmethod
    def generate_square_subsequent_mask(length):
        return as_tensor(torch.triu(torch.full((length, length), float("-inf"), device=_dt.default_device()), 1))


# ------------------------------------------------------------------ recurrent (wrapping torch cells)
class _RNNBase(Layer):
    _mode = "LSTM"

    def __init__(self, input_size, hidden_size, num_layers=1, direction="forward", time_major=False, dropout=0.0,
                 weight_ih_attr=None, weight_hh_attr=None, bias_ih_attr=None, bias_hh_attr=None, name=None, **kw):
        super().__init__()
        bi = direction in ("bidirect", "bidirectional")
        cls = {"LSTM": torch.nn.LSTM, "GRU": torch.nn.GRU, "RNN": torch.nn.RNN}[self._mode]
        self._impl = cls(input_size, hidden_size, num_layers, batch_first=not time_major, dropout=dropout,
                         bidirectional=bi).to(_dt.default_device())
        for n, p in self._impl.named_parameters():
            self.add_parameter(n, EagerParamBase(p.data, True))
        self._names = [n for n, _ in self._impl.named_parameters()]

    def forward(self, inputs, initial_states=None, sequence_length=None):
        if sequence_length is not None:
            return self._forward_lengths(inputs, initial_states, sequence_length)
        params = {n: self._parameters[n] for n in self._names}
        out, st = torch.func.functional_call(self._impl, params, (inputs, initial_states))
        return out, st

    def _forward_lengths(self, inputs, initial_states, sequence_length):
        """Padded steps leave the state untouched and give zero output (python/paddle/nn/layer/rnn.py:1560-1640):
        the stepped form of the ``rnn`` operator."""
        from ..._op_table_seq import rnn
        impl = self._impl
        dirs = 2 if impl.bidirectional else 1
        x = inputs if not impl.batch_first else inputs.transpose([1, 0, 2])
        B = x.shape[1]
        mode = {"LSTM": "LSTM", "GRU": "GRU", "RNN": "RNN_TANH" if getattr(impl, "nonlinearity", "tanh") == "tanh" else "RNN_RELU"}[self._mode]
        if initial_states is None:
            z = torch.zeros(impl.num_layers * dirs, B, impl.hidden_size, dtype=x.dtype, device=x.device)
            initial_states = (z, z.clone()) if mode == "LSTM" else z
        states = list(initial_states) if isinstance(initial_states, (list, tuple)) else [initial_states]
        sfx = [""] + (["_reverse"] if dirs == 2 else [])
        mats, biases = [], []
        for layer in range(impl.num_layers):
            for s in sfx:
                mats += [self._parameters[f"weight_ih_l{layer}{s}"], self._parameters[f"weight_hh_l{layer}{s}"]]
                if impl.bias:
                    biases += [self._parameters[f"bias_ih_l{layer}{s}"], self._parameters[f"bias_hh_l{layer}{s}"]]
        out, _, final, _ = rnn(x, states, mats + biases, sequence_length, None, impl.dropout, impl.bidirectional, impl.input_size,
                               impl.hidden_size, impl.num_layers, mode, 0, not self.training)
        if impl.batch_first:
            out = out.transpose([1, 0, 2])
        return out, (tuple(final) if mode == "LSTM" else final[0])


class LSTM(_RNNBase):
    _mode = "LSTM"


class GRU(_RNNBase):
    _mode = "GRU"


class SimpleRNN(_RNNBase):
    _mode = "RNN"
