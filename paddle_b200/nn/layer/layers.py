"""``paddle.nn.Layer``: module base class with Paddle's semantics.

Re-implements the behaviour of python/paddle/nn/layer/layers.py: parameter / sublayer / buffer
registries, ``create_parameter`` with ParamAttr and the ``<layer>_<n>.w_<m>`` naming scheme
(python/paddle/base/layer_helper_base.py:373-391), forward pre/post hooks
(``register_forward_pre_hook:698``), ``state_dict`` keyed by structured names (``:1979``),
``set_state_dict`` (``:2126``), ``to``/``astype`` casts (``:2429``), train/eval flags.
"""
from __future__ import annotations

import collections
import re
from typing import Callable, Iterator

import numpy as np
import torch

from ..._core import dtype as _dt
from ..._core import unique_name
from ..._core.tensor import EagerParamBase, Tensor, as_tensor, to_tensor


class ParamAttr:
    """python/paddle/base/param_attr.py"""

    def __init__(self, name=None, initializer=None, learning_rate=1.0, regularizer=None, trainable=True,
                 do_model_average=True, need_clip=True):
        self.name = name
        self.initializer = initializer
        self.learning_rate = learning_rate
        self.regularizer = regularizer
        self.trainable = trainable
        self.do_model_average = do_model_average
        self.need_clip = need_clip

    @staticmethod
    def _to_attr(arg):
        if arg is None:
            return ParamAttr()
        if isinstance(arg, ParamAttr):
            return arg
        if isinstance(arg, str):
            return ParamAttr(name=arg)
        if isinstance(arg, bool):
            return ParamAttr() if arg else False
        if callable(arg) or hasattr(arg, "__call__"):
            return ParamAttr(initializer=arg)
        raise TypeError(f"cannot interpret {arg!r} as ParamAttr")


class HookRemoveHelper:
    _next_id = 0

    def __init__(self, hooks):
        self._hooks = hooks
        self._id = HookRemoveHelper._next_id
        HookRemoveHelper._next_id += 1

    def remove(self):
        self._hooks.pop(self._id, None)


def _camel_to_snake(name: str) -> str:
    s1 = re.sub("(.)([A-Z][a-z]+)", r"\1_\2", name)
    return re.sub("([a-z0-9])([A-Z])", r"\1_\2", s1).lower()


class Layer:
    def __init__(self, name_scope=None, dtype="float32"):
        d = self.__dict__
        d["training"] = True
        d["_parameters"] = collections.OrderedDict()
        d["_sub_layers"] = collections.OrderedDict()
        d["_buffers"] = collections.OrderedDict()
        d["_non_persistable_buffer_names_set"] = set()
        d["_forward_pre_hooks"] = collections.OrderedDict()
        d["_forward_post_hooks"] = collections.OrderedDict()
        d["_dtype"] = _dt.to_torch(dtype) if dtype is not None else _dt.get_default_dtype()
        if name_scope is None:
            name_scope = _camel_to_snake(self.__class__.__name__)
        d["_full_name"] = unique_name.generate(name_scope)
        d["_param_counter"] = collections.defaultdict(int)
        d["_casted_by_pure_fp16"] = False

    # ------------------------------------------------------------------ naming / creation
    def full_name(self):
        return self._full_name

    def __init_subclass__(cls, **kw):
        # Layer construction (parameter/buffer creation and initialisation) is never part of a recorded static
        # program: the reference puts those ops in the startup program, here they simply run once, eagerly.
        super().__init_subclass__(**kw)
        init = cls.__dict__.get("__init__")
        if init is not None:
            from ...static.graph import no_trace
            cls.__init__ = no_trace(init)

    def create_parameter(self, shape, attr=None, dtype=None, is_bias=False, default_initializer=None):
        from ...static.graph import suspend
        with suspend():
            return self._create_parameter(shape, attr, dtype, is_bias, default_initializer)

    def _create_parameter(self, shape, attr=None, dtype=None, is_bias=False, default_initializer=None):
        from ..initializer import Constant, XavierUniform, _global_initializer
        attr = ParamAttr._to_attr(attr)
        if attr is False:
            return None
        td = _dt.to_torch(dtype) if dtype is not None else self._dtype
        suffix = "b" if is_bias else "w"
        name = attr.name or unique_name.generate(".".join([self._full_name, suffix]))
        data = torch.empty(tuple(int(s) for s in shape), dtype=td, device=_dt.default_device())
        p = EagerParamBase(data, trainable=attr.trainable, name=name)
        p.optimize_attr = {"learning_rate": attr.learning_rate}
        p.regularizer = attr.regularizer
        p.need_clip = attr.need_clip
        p.do_model_average = attr.do_model_average
        init = attr.initializer or default_initializer or _global_initializer(is_bias)
        if init is None:
            init = Constant(0.0) if is_bias else XavierUniform()
        from ... import _lazy_init_active
        if _lazy_init_active():
            # under ``paddle.LazyGuard`` the values are not computed yet: ``param.initialize()`` runs the initializer
            # (the storage is reserved but untouched, so no pages are committed until then)
            p._deferred_init = init
            return p
        with torch.no_grad():
            init(p)
        return p

    def create_variable(self, name=None, persistable=None, dtype=None):
        t = as_tensor(torch.empty(0, dtype=_dt.to_torch(dtype) or self._dtype, device=_dt.default_device()))
        if name:
            t.name = name
        return t

    create_tensor = create_variable

    # ------------------------------------------------------------------ registries
    def add_parameter(self, name, parameter):
        if parameter is not None and not isinstance(parameter, EagerParamBase):
            raise TypeError("add_parameter expects a Parameter")
        self._parameters[name] = parameter
        return parameter

    def add_sublayer(self, name, sublayer):
        self._sub_layers[str(name)] = sublayer
        return sublayer

    def register_buffer(self, name, tensor, persistable=True):
        if tensor is not None and not isinstance(tensor, torch.Tensor):
            raise TypeError("register_buffer expects a Tensor")
        self._buffers[name] = None if tensor is None else as_tensor(tensor)
        if not persistable:
            self._non_persistable_buffer_names_set.add(name)
        else:
            self._non_persistable_buffer_names_set.discard(name)

    def __setattr__(self, name, value):
        d = self.__dict__
        if isinstance(value, EagerParamBase):
            for reg in ("_sub_layers", "_buffers"):
                d.get(reg, {}).pop(name, None)
            d.pop(name, None)
            d["_parameters"][name] = value
        elif isinstance(value, Layer):
            for reg in ("_parameters", "_buffers"):
                d.get(reg, {}).pop(name, None)
            d.pop(name, None)
            d["_sub_layers"][name] = value
        elif "_parameters" in d and name in d["_parameters"]:
            if value is not None and not isinstance(value, torch.Tensor):
                raise TypeError(f"cannot assign {type(value)} to parameter {name}")
            if value is None:
                d["_parameters"][name] = None
            else:
                d["_parameters"][name].set_value(value)
        elif "_buffers" in d and name in d["_buffers"]:
            d["_buffers"][name] = None if value is None else as_tensor(value)
        elif "_sub_layers" in d and name in d["_sub_layers"]:
            d["_sub_layers"][name] = value
        else:
            object.__setattr__(self, name, value)

    def __getattr__(self, name):
        d = self.__dict__
        for reg in ("_parameters", "_sub_layers", "_buffers"):
            r = d.get(reg)
            if r is not None and name in r:
                return r[name]
        raise AttributeError(f"'{type(self).__name__}' object has no attribute '{name}'")

    def __delattr__(self, name):
        for reg in ("_parameters", "_sub_layers", "_buffers"):
            if name in self.__dict__[reg]:
                del self.__dict__[reg][name]
                return
        object.__delattr__(self, name)

    def __dir__(self):
        return list(super().__dir__()) + list(self._parameters) + list(self._sub_layers) + list(self._buffers)

    # ------------------------------------------------------------------ traversal
    def named_sublayers(self, prefix="", include_self=False, layers_set=None, remove_duplicate=True) -> Iterator:
        layers_set = set() if layers_set is None else layers_set
        if include_self and id(self) not in layers_set:
            layers_set.add(id(self))
            yield prefix, self
        for key, layer in self._sub_layers.items():
            if layer is None or id(layer) in layers_set:
                continue
            p = prefix + ("." if prefix else "") + key
            layers_set.add(id(layer))
            yield p, layer
            yield from layer.named_sublayers(p, False, layers_set)

    def sublayers(self, include_self=False):
        return [l for _, l in self.named_sublayers(include_self=include_self)]

    def children(self):
        return iter(l for l in self._sub_layers.values() if l is not None)

    def named_children(self):
        return iter((n, l) for n, l in self._sub_layers.items() if l is not None)

    def named_parameters(self, prefix="", include_sublayers=True):
        seen = set()
        layers = self.named_sublayers(prefix, include_self=True) if include_sublayers else [(prefix, self)]
        for lp, layer in layers:
            for k, p in layer._parameters.items():
                if p is None or id(p) in seen:
                    continue
                seen.add(id(p))
                yield lp + ("." if lp else "") + k, p

    def parameters(self, include_sublayers=True):
        return [p for _, p in self.named_parameters(include_sublayers=include_sublayers)]

    def named_buffers(self, prefix="", include_sublayers=True):
        seen = set()
        layers = self.named_sublayers(prefix, include_self=True) if include_sublayers else [(prefix, self)]
        for lp, layer in layers:
            for k, b in layer._buffers.items():
                if b is None or id(b) in seen:
                    continue
                seen.add(id(b))
                yield lp + ("." if lp else "") + k, b

    def buffers(self, include_sublayers=True):
        return [b for _, b in self.named_buffers(include_sublayers=include_sublayers)]

    def apply(self, fn: Callable):
        for l in self.children():
            l.apply(fn)
        fn(self)
        return self

    # ------------------------------------------------------------------ mode / call
    def train(self):
        for l in self.sublayers(include_self=True):
            l.__dict__["training"] = True
        return self

    def eval(self):
        for l in self.sublayers(include_self=True):
            l.__dict__["training"] = False
        return self

    def register_forward_pre_hook(self, hook):
        h = HookRemoveHelper(self._forward_pre_hooks)
        self._forward_pre_hooks[h._id] = hook
        return h

    def register_forward_post_hook(self, hook):
        h = HookRemoveHelper(self._forward_post_hooks)
        self._forward_post_hooks[h._id] = hook
        return h

    def forward(self, *inputs, **kwargs):
        raise NotImplementedError

    def __call__(self, *inputs, **kwargs):
        for hook in list(self._forward_pre_hooks.values()):
            r = hook(self, inputs)
            if r is not None:
                inputs = r if isinstance(r, tuple) else (r,)
        out = self.forward(*inputs, **kwargs)
        for hook in list(self._forward_post_hooks.values()):
            r = hook(self, inputs, out)
            if r is not None:
                out = r
        return out

    # ------------------------------------------------------------------ state dict
    def state_dict(self, destination=None, include_sublayers=True, structured_name_prefix="", use_hook=True,
                   keep_vars=True):
        dest = collections.OrderedDict() if destination is None else destination
        for name, p in self.named_parameters(structured_name_prefix.rstrip("."), include_sublayers):
            dest[name] = p
        layers = self.named_sublayers(structured_name_prefix.rstrip("."), include_self=True) if include_sublayers \
            else [(structured_name_prefix.rstrip("."), self)]
        for lp, layer in layers:
            for k, b in layer._buffers.items():
                if b is not None and k not in layer._non_persistable_buffer_names_set:
                    dest[lp + ("." if lp else "") + k] = b
        return dest

    def to_static_state_dict(self, *a, **k):
        return self.state_dict(*a, **k)

    def set_state_dict(self, state_dict, use_structured_name=True):
        own = self.state_dict()
        if not use_structured_name:
            own = {v.name: v for v in own.values()}
        missing, unexpected = [], []
        for k, target in own.items():
            if k not in state_dict:
                missing.append(k)
                continue
            v = state_dict[k]
            if isinstance(v, np.ndarray):
                v = to_tensor(v)
            elif not isinstance(v, torch.Tensor):
                v = to_tensor(np.asarray(v))
            if list(v.shape) != list(target.shape):
                raise ValueError(f"shape mismatch for {k}: checkpoint {list(v.shape)} vs layer {list(target.shape)}")
            with torch.no_grad():
                target.data.copy_(v.to(target.dtype))
        for k in state_dict:
            if k not in own and not str(k).endswith("@@"):
                unexpected.append(k)
        return missing, unexpected

    set_dict = set_state_dict
    load_dict = set_state_dict

    # ------------------------------------------------------------------ casts / movement
    def _apply_to_tensors(self, fn, floating_only=True):
        for layer in self.sublayers(include_self=True):
            for k, p in layer._parameters.items():
                if p is None:
                    continue
                if floating_only and not p.is_floating_point():
                    continue
                new = fn(p.data)
                if new is not p.data:
                    if p.requires_grad and not (new.is_floating_point() or new.is_complex()):
                        p.requires_grad_(False)           # integer parameters cannot take gradients
                    p.data = new
                if p.grad is not None:
                    p.grad = fn(p.grad)
            for k, b in layer._buffers.items():
                if b is None or (floating_only and not b.is_floating_point()):
                    continue
                layer._buffers[k] = as_tensor(fn(b))

    def to(self, device=None, dtype=None, blocking=None):
        dev = _dt.to_device(device)
        td = _dt.to_torch(dtype)
        if dev is not None:
            self._apply_to_tensors(lambda t: t.to(dev), floating_only=False)
        if td is not None:
            self._apply_to_tensors(lambda t: t.to(td))
            for l in self.sublayers(include_self=True):
                l.__dict__["_dtype"] = td
        return self

    def astype(self, dtype):
        return self.to(dtype=dtype)

    def float(self, excluded_layers=None):
        return self._cast_excluding(torch.float32, excluded_layers)

    def float16(self, excluded_layers=None):
        return self._cast_excluding(torch.float16, excluded_layers)

    def bfloat16(self, excluded_layers=None):
        return self._cast_excluding(torch.bfloat16, excluded_layers)

    def _cast_excluding(self, td, excluded_layers):
        excl = tuple(excluded_layers) if isinstance(excluded_layers, (list, tuple)) else (
            (excluded_layers,) if excluded_layers else ())
        for layer in self.sublayers(include_self=True):
            if excl and isinstance(layer, excl):
                continue
            for p in layer._parameters.values():
                if p is not None and p.is_floating_point():
                    p.data = p.data.to(td)
            for k, b in layer._buffers.items():
                if b is not None and b.is_floating_point():
                    layer._buffers[k] = as_tensor(b.to(td))
            layer.__dict__["_dtype"] = td
        return self

    def cuda(self, device=None):
        return self.to(device=f"gpu:{device}" if isinstance(device, int) else (device or "gpu"))

    def cpu(self):
        return self.to(device="cpu")

    def clear_gradients(self, set_to_zero=True):
        for p in self.parameters():
            p.clear_gradient(set_to_zero)

    def extra_repr(self):
        return ""

    def __repr__(self):
        lines = []
        for k, l in self._sub_layers.items():
            sub = repr(l).split("\n")
            lines.append(f"  ({k}): " + "\n  ".join(sub))
        head = f"{type(self).__name__}({self.extra_repr()}"
        return head + ("\n" + "\n".join(lines) + "\n)" if lines else ")")
