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
    """Holds a quanter / observer class with its arguments; one instance is made per quantised layer."""

    def __init__(self, cls, _shown_name=None, **kw):
        self._cls, self._kw = cls, kw
        self._shown_name = _shown_name or cls.__name__

    def _instance(self, layer=None):
        return self._cls(**self._kw)

    def __repr__(self):
        return f"{self._shown_name}(" + ",".join(f"{k}={v}" for k, v in self._kw.items()) + ")"

    __str__ = __repr__


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
    return _Factory(FakeQuanterWithAbsMaxObserverLayer, "FakeQuanterWithAbsMaxObserver", name=name, moving_rate=moving_rate,
                    bit_length=bit_length, dtype=dtype)


class quanters:
    FakeQuanterWithAbsMaxObserver = staticmethod(FakeQuanterWithAbsMaxObserver)


class observers:
    AbsmaxObserver = staticmethod(lambda quant_bits=8: _Factory(AbsmaxObserver, quant_bits=quant_bits))


class SingleLayerConfig:
    """Activation and weight quanter factories of one layer (python/paddle/quantization/config.py)."""

    def __init__(self, activation, weight):
        self._activation, self._weight = activation, weight

    activation = property(lambda self: self._activation)
    weight = property(lambda self: self._weight)

    def __iter__(self):                       # unpacks like the (activation, weight) pair it replaces
        return iter((self._activation, self._weight))

    def __str__(self):
        return f"activation: {self._activation}\nweight: {self._weight}"


SingleLayerConfig.__module__ = "paddle.quantization.config"


class QuantConfig:
    """Which layers are quantised and how: a global default, overridden by layer type, by layer-name prefix and by
    layer instance (most specific wins); ``add_qat_layer_mapping`` names the quantised stand-in of a layer type and
    ``add_customized_leaf`` marks container types that are quantised as a whole."""

    def __init__(self, activation=None, weight=None):
        self._global_config = SingleLayerConfig(activation, weight) if (activation is not None or weight is not None) else None
        self._global = (activation, weight)
        self._by_type, self._by_layer, self._by_name = {}, {}, {}
        self._layer2config = {}
        self._qat_layer_mapping = {}
        self._customized_leaves = []

    def add_type_config(self, layer_type, activation=None, weight=None):
        for t in (layer_type if isinstance(layer_type, (list, tuple)) else [layer_type]):
            self._by_type[t] = SingleLayerConfig(activation, weight)

    def add_layer_config(self, layer, activation=None, weight=None):
        for l in (layer if isinstance(layer, (list, tuple)) else [layer]):
            self._by_layer[id(l)] = SingleLayerConfig(activation, weight)
            self._by_name.setdefault(l.full_name(), self._by_layer[id(l)])
            self._shown_prefix = getattr(self, "_shown_prefix", {})
            self._shown_prefix[l.full_name()] = self._by_layer[id(l)]

    def add_name_config(self, layer_name, activation=None, weight=None):
        for n in (layer_name if isinstance(layer_name, (list, tuple)) else [layer_name]):
            self._by_name[n] = SingleLayerConfig(activation, weight)
            self._shown_prefix = getattr(self, "_shown_prefix", {})
            self._shown_prefix[n] = self._by_name[n]

    def add_qat_layer_mapping(self, source, target):
        """Layers of type ``source`` are replaced by ``target(layer, config)`` in quantisation-aware training."""
        if not (isinstance(source, type) and isinstance(target, type)):
            raise TypeError("The source layer and the target layer should be classes (subclasses of paddle.nn.Layer)")
        self._qat_layer_mapping[source] = target

    def add_customized_leaf(self, layer_type):
        self._customized_leaves.append(layer_type)

    customized_leaves = property(lambda self: self._customized_leaves)
    qat_layer_mappings = property(lambda self: self._qat_layer_mapping)
    global_config = property(lambda self: self._global_config)

    def _is_leaf(self, layer):
        return not list(layer.children()) or any(isinstance(layer, t) for t in self._customized_leaves)

    def _specify(self, model):
        """Resolve the configuration of every leaf layer of ``model`` (kept in ``_layer2config``)."""
        self._layer2config = {}
        for name, sub in model.named_sublayers(include_self=True):
            if not self._is_leaf(sub):
                continue
            cfg = self._lookup(name, sub)
            if cfg is not None:
                self._layer2config[sub] = cfg if isinstance(cfg, SingleLayerConfig) else SingleLayerConfig(*cfg)
        return self._layer2config

    def _get_config_by_layer(self, layer):
        return self._layer2config.get(layer)

    def _is_quantifiable(self, layer):
        return layer in self._layer2config

    def __str__(self):
        out = "Global config:\n" + (str(self._global_config) if self._global_config is not None else "None")
        if self._by_type:
            out += f"\nLayer type config:\n{self._by_type}"
        if getattr(self, "_shown_prefix", None):
            out += f"\nLayer prefix config:\n{self._shown_prefix}"
        return out

    def _lookup(self, name, layer):
        if id(layer) in self._by_layer:
            return self._by_layer[id(layer)]
        if name in self._by_name:
            return self._by_name[name]
        full = layer.full_name() if hasattr(layer, "full_name") else None
        for prefix, cfg in self._by_name.items():
            if full is not None and full.startswith(prefix):
                return cfg
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


# ``paddle.quantization.quanters`` / ``observers`` / ``config`` ... are modules in the reference
import sys as _sys  # noqa: E402
import types as _types  # noqa: E402


def _as_module(ns, name):
    m = _types.ModuleType(name)
    for k, v in vars(ns).items():
        if not k.startswith("__"):
            setattr(m, k, v.__func__ if isinstance(v, staticmethod) else v)
    _sys.modules[name] = m
    return m


quanters = _as_module(quanters, __name__ + ".quanters")
observers = _as_module(observers, __name__ + ".observers")
from .._core.submodule_alias import alias_submodules as _alias  # noqa: E402
_alias(__name__, ("config", "ptq", "qat", "quantize", "base_observer", "base_quanter", "factory", "wrapper"))
