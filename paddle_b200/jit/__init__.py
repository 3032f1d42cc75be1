"""``paddle.jit``: dynamic-to-static capture (python/paddle/jit/api.py:197 ``to_static``, :956 ``save``,
:1527 ``load``; dy2static/program_translator.py:398 ``StaticFunction``, :1614 ``ProgramCache``).

The reference traces Python into a PIR program executed by its interpreter.  Here the captured artefact is a
CUDA graph: a ``StaticFunction`` keeps a cache keyed by the input signature (the guards: shapes, dtypes,
training flag, grad mode); for a grad-free call on GPU the first hit warms up, the second captures the whole
function into one CUDA graph with static input/output buffers, later hits copy inputs in and replay — one
launch per call instead of one per operator.  Calls that need autograd (training) run eagerly through the
same cache entry, so semantics never depend on whether a graph exists.
"""
from __future__ import annotations

import os
import pickle

import torch

from .._core.tensor import as_tensor
from ..nn.layer.layers import Layer
from ..static import InputSpec

_to_static_enabled = True


def enable_to_static(flag: bool):
    global _to_static_enabled
    _to_static_enabled = bool(flag)


def ignore_module(modules):
    pass


def not_to_static(fn=None):
    if fn is not None:
        fn._not_to_static = True
    return fn


class _CacheEntry:
    def __init__(self):
        self.calls = 0
        self.graph = None
        self.static_in = None
        self.static_out = None


class ProgramCache(dict):
    def concrete_programs(self):
        return list(self.values())


def _flatten(obj, out):
    if isinstance(obj, torch.Tensor):
        out.append(obj)
    elif isinstance(obj, (list, tuple)):
        for o in obj:
            _flatten(o, out)
    elif isinstance(obj, dict):
        for o in obj.values():
            _flatten(o, out)
    return out


def _rebuild(template, it):
    if isinstance(template, torch.Tensor):
        return as_tensor(next(it))
    if isinstance(template, (list, tuple)):
        return type(template)(_rebuild(t, it) for t in template)
    if isinstance(template, dict):
        return {k: _rebuild(v, it) for k, v in template.items()}
    return template


class StaticFunction:
    def __init__(self, function, input_spec=None, build_strategy=None, backend=None, full_graph=False, layer=None):
        self._fn = function
        self._layer = layer
        self._input_spec = list(input_spec) if input_spec is not None else None
        self._cache = ProgramCache()
        self._use_cuda_graph = True
        self.__name__ = getattr(function, "__name__", "static_fn")

    @property
    def program_cache(self):
        return self._cache

    @property
    def dygraph_function(self):
        return self._fn

    def rollback(self):
        return self._fn

    def get_concrete_program(self, *args, **kwargs):
        return self._key(args, kwargs), self._cache.get(self._key(args, kwargs))

    concrete_program = property(lambda self: next(iter(self._cache.values()), None))

    def __get__(self, instance, owner):
        if instance is None:
            return self
        bound = StaticFunction(self._fn.__get__(instance, owner), self._input_spec, layer=instance)
        bound._cache = instance.__dict__.setdefault("_jit_caches", {}).setdefault(self.__name__, ProgramCache())
        return bound

    def _key(self, args, kwargs):
        tensors = _flatten((args, kwargs), [])
        training = self._layer.training if isinstance(self._layer, Layer) else None
        return (tuple((tuple(t.shape), t.dtype, t.device.type) for t in tensors), training, torch.is_grad_enabled(),
                tuple(a for a in args if isinstance(a, (int, float, str, bool, type(None)))))

    def _check_spec(self, args):
        if self._input_spec is None:
            return
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        for spec, t in zip(self._input_spec, tensors):
            if isinstance(spec, InputSpec) and not spec.matches(t):
                raise ValueError(f"input {tuple(t.shape)}/{t.dtype} does not match {spec}")

    def __call__(self, *args, **kwargs):
        if not _to_static_enabled:
            return self._fn(*args, **kwargs)
        self._check_spec(args)
        key = self._key(args, kwargs)
        entry = self._cache.get(key)
        if entry is None:
            entry = self._cache[key] = _CacheEntry()
        entry.calls += 1
        tensors = _flatten((args, kwargs), [])
        needs_grad = torch.is_grad_enabled() and (
            any(t.requires_grad for t in tensors)
            or (isinstance(self._layer, Layer) and any(p.requires_grad for p in self._layer.parameters())))
        on_gpu = bool(tensors) and all(t.is_cuda for t in tensors)
        if needs_grad or not on_gpu or not self._use_cuda_graph:
            return self._fn(*args, **kwargs)
        if entry.graph is None:
            if entry.calls < 2:       # first call: eager warm-up (lazy initialisation, autotuning, allocations)
                return self._fn(*args, **kwargs)
            try:
                self._capture(entry, args, kwargs, tensors)
            except Exception:  # noqa: BLE001 - functions with host syncs cannot be captured: stay eager
                entry.graph = False
                torch.cuda.synchronize()
                return self._fn(*args, **kwargs)
        if entry.graph is False:
            return self._fn(*args, **kwargs)
        for dst, src in zip(entry.static_in, tensors):
            dst.copy_(src)
        entry.graph.replay()
        outs = [o.clone() for o in entry.static_out_flat]
        return _rebuild(entry.static_out, iter(outs))

    def _capture(self, entry, args, kwargs, tensors):
        entry.static_in = [t.detach().clone() for t in tensors]
        it = iter(entry.static_in)
        s_args, s_kwargs = _rebuild((args, kwargs), it)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._fn(*s_args, **s_kwargs)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = self._fn(*s_args, **s_kwargs)
        entry.graph = g
        entry.static_out = out
        entry.static_out_flat = _flatten(out, [])


def to_static(function=None, input_spec=None, build_strategy=None, backend=None, full_graph=False, **kwargs):
    def decorate(fn):
        if full_graph:
            # whole-graph conversion: Python control flow on tensors becomes cond / while_loop nodes of a recorded
            # static program that is replayed on later calls (dy2static.py)
            from .dy2static import ProgramFunction
            if isinstance(fn, Layer):
                fn.__dict__["forward"] = ProgramFunction(fn.forward, fn)
                return fn
            return ProgramFunction(fn)
        if isinstance(fn, Layer):
            layer = fn
            sf = StaticFunction(layer.forward, input_spec, layer=layer)
            layer.__dict__["forward"] = sf
            return layer
        return StaticFunction(fn, input_spec, build_strategy, backend, full_graph)
    if function is not None:
        return decorate(function)
    return decorate


class TranslatedLayer(Layer):
    """A layer restored by :func:`load`."""

    def __init__(self, inner):
        super().__init__()
        self._inner = inner

    def forward(self, *args, **kwargs):
        return self._inner(*args, **kwargs)

    def program(self):
        return None


def save(layer, path, input_spec=None, **configs):
    """Writes ``<path>.pdiparams`` (parameters in the ``paddle.save`` state-dict format), ``<path>.pdmodel``
    (the pickled layer structure without parameter data) and ``<path>.pdiparams.info`` (input specs)."""
    import cloudpickle

    from ..framework.io import save as _save
    d = os.path.dirname(path)
    if d:
        os.makedirs(d, exist_ok=True)
    inner = layer
    fwd = inner.__dict__.pop("forward", None) if isinstance(inner, Layer) else None
    try:
        _save(inner.state_dict(), path + ".pdiparams")
        with open(path + ".pdmodel", "wb") as f:
            cloudpickle.dump(inner, f)
        with open(path + ".pdiparams.info", "wb") as f:
            pickle.dump({"input_spec": [repr(s) for s in (input_spec or [])]}, f)
    finally:
        if fwd is not None:
            inner.__dict__["forward"] = fwd


def load(path, **configs):
    from ..framework.io import load as _load
    with open(path + ".pdmodel", "rb") as f:
        inner = pickle.load(f)
    inner.set_state_dict(_load(path + ".pdiparams"))
    inner.eval()
    return TranslatedLayer(inner)


def set_code_level(level=100, also_to_stdout=False):
    pass


def set_verbosity(level=0, also_to_stdout=False):
    pass


class marker:
    @staticmethod
    def unified(fn):
        return fn
