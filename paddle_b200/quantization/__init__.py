"""``paddle.quantization`` (python/paddle/quantization/): ``QuantConfig`` + ``QAT`` / ``PTQ`` drivers, observers and
fake quanters.  ``QAT.quantize`` wraps the configured layers so that weights and activations pass through a
straight-through fake-quantisation; ``PTQ`` collects ranges with observers; ``convert`` folds the learned scales into
plain attributes (``weight_scale`` / ``activation_scale``)."""
from __future__ import annotations

import copy

import torch

from .._core.tensor import as_tensor
from ..nn.layer.layers import Layer


class _STEQuant(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, bits):
        q = 2 ** (bits - 1) - 1
        s = scale.clamp(min=1e-8) / q
        return torch.round(x / s).clamp(-q, q) * s

    @staticmethod
    def backward(ctx, g):
        return g, None, None


class BaseObserver(Layer):
    def __init__(self, quant_bits=8):
        super().__init__()
        self._bits = quant_bits
        self._scale = None

    def forward(self, x):
        self._observe(x.detach())
        return x

    def scales(self):
        return as_tensor(self._scale) if self._scale is not None else None

    def bit_length(self):
        return self._bits

    def quant_axis(self):
        return -1

    def zero_points(self):
        return None


class AbsmaxObserver(BaseObserver):
    def _observe(self, x):
        m = x.abs().max().float()
        self._scale = m if self._scale is None else torch.maximum(self._scale, m)


class _Factory:
    def __init__(self, cls, **kw):
        self._cls, self._kw = cls, kw

    def _instance(self, layer=None):
        return self._cls(**self._kw)


class FakeQuanterWithAbsMaxObserverLayer(BaseObserver):
    def __init__(self, moving_rate=0.9, bit_length=8, dtype="float32", name=None):
        super().__init__(bit_length)
        self._rate = moving_rate

    def forward(self, x):
        m = x.detach().abs().max().float()
        if self.training or self._scale is None:
            self._scale = m if self._scale is None else self._rate * self._scale + (1 - self._rate) * m
        return as_tensor(_STEQuant.apply(x, self._scale.to(x.dtype), self._bits))


def FakeQuanterWithAbsMaxObserver(moving_rate=0.9, bit_length=8, dtype="float32", name=None):
    return _Factory(FakeQuanterWithAbsMaxObserverLayer, moving_rate=moving_rate, bit_length=bit_length)


class quanters:
    FakeQuanterWithAbsMaxObserver = staticmethod(FakeQuanterWithAbsMaxObserver)


class observers:
    AbsmaxObserver = staticmethod(lambda quant_bits=8: _Factory(AbsmaxObserver, quant_bits=quant_bits))


class QuantConfig:
    def __init__(self, activation=None, weight=None):
        self._global = (activation, weight)
        self._by_type, self._by_layer, self._by_name = {}, {}, {}

    def add_type_config(self, layer_type, activation=None, weight=None):
        for t in (layer_type if isinstance(layer_type, (list, tuple)) else [layer_type]):
            self._by_type[t] = (activation, weight)

    def add_layer_config(self, layer, activation=None, weight=None):
        for l in (layer if isinstance(layer, (list, tuple)) else [layer]):
            self._by_layer[id(l)] = (activation, weight)

    def add_name_config(self, layer_name, activation=None, weight=None):
        for n in (layer_name if isinstance(layer_name, (list, tuple)) else [layer_name]):
            self._by_name[n] = (activation, weight)

    def _lookup(self, name, layer):
        if id(layer) in self._by_layer:
            return self._by_layer[id(layer)]
        if name in self._by_name:
            return self._by_name[name]
        for t, cfg in self._by_type.items():
            if isinstance(layer, t):
                return cfg
        from ..nn import Conv2D, Linear
        if isinstance(layer, (Linear, Conv2D)) and any(c is not None for c in self._global):
            return self._global
        return None


class QuantedLayer(Layer):
    """Wrapper produced by ``quantize``: observes / fake-quantises the input and the wrapped layer's weight."""

    def __init__(self, inner, act_q, w_q):
        super().__init__()
        self.inner, self.activation_quanter, self.weight_quanter = inner, act_q, w_q

    def forward(self, x):
        if self.activation_quanter is not None:
            x = self.activation_quanter(x)
        if self.weight_quanter is None or getattr(self.inner, "weight", None) is None:
            return self.inner(x)
        w = self.inner.weight
        saved = w.data
        try:
            qw = self.weight_quanter(w)
            if qw is not w:
                self.inner._parameters["weight"] = qw
            return self.inner(x)
        finally:
            self.inner._parameters["weight"] = w
            w.data = saved


class _Quantization:
    def __init__(self, config: QuantConfig):
        self._config = config

    def quantize(self, model, inplace=False):
        model = model if inplace else copy.deepcopy(model)
        for name, sub in list(model.named_sublayers()):
            cfg = self._config._lookup(name, sub)
            if cfg is None or isinstance(sub, QuantedLayer):
                continue
            act, w = cfg
            wrapped = QuantedLayer(sub, act._instance(sub) if act else None, w._instance(sub) if w else None)
            parent, key = model, name
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            parent._sub_layers[parts[-1]] = wrapped
        return model

    def convert(self, model, inplace=False, remain_weight=False):
        model = model if inplace else copy.deepcopy(model)
        for name, sub in list(model.named_sublayers()):
            if isinstance(sub, QuantedLayer):
                inner = sub.inner
                inner.weight_scale = sub.weight_quanter.scales() if sub.weight_quanter is not None else None
                inner.activation_scale = sub.activation_quanter.scales() if sub.activation_quanter is not None else None
                parent = model
                parts = name.split(".")
                for p in parts[:-1]:
                    parent = getattr(parent, p)
                parent._sub_layers[parts[-1]] = inner
        return model


class QAT(_Quantization):
    pass


class PTQ(_Quantization):
    pass


class BaseQuanter(BaseObserver):
    """Base class of trainable quantizers (python/paddle/quantization/base_quanter.py)."""


def quanter(class_name):
    """Class decorator that registers a quanter layer and creates a factory of the given name in the caller's module
    (python/paddle/quantization/factory.py ``quanter``)."""
    import sys

    def wrapper(target_class):
        def init(self, *args, **kwargs):
            self._args, self._kwargs = args, kwargs

        def _instance(self, layer=None):
            return target_class(*self._args, **self._kwargs)
        factory = type(class_name, (_Factory,), {"__init__": init, "_instance": _instance, "_get_class": lambda self: target_class})
        mod = sys.modules[target_class.__module__]
        setattr(mod, class_name, factory)
        return target_class
    return wrapper
