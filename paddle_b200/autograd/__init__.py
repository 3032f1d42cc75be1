"""``paddle.autograd``: PyLayer, backward, grad, saved-tensor hooks, jacobian/hessian
(python/paddle/autograd/py_layer.py, backward_mode.py:140, autograd.py) on torch.autograd."""
from __future__ import annotations

import contextlib

import torch

from .._core.tensor import Tensor, as_tensor


class PyLayerContext:
    """Kept for isinstance checks; the live context object is torch's FunctionCtx, which already offers
    ``save_for_backward`` and ``needs_input_grad``.  ``saved_tensor()`` is added below."""


def _saved_tensor(self):
    return self.saved_tensors


torch.autograd.function.FunctionCtx.saved_tensor = _saved_tensor
torch.autograd.function.FunctionCtx.mark_not_inplace = lambda self, *a: None
torch.autograd.function.FunctionCtx.set_materialize_grads = (
    torch.autograd.function.FunctionCtx.set_materialize_grads)


class PyLayer(torch.autograd.Function):
    """User-defined differentiable op: ``forward(ctx, *args)`` / ``backward(ctx, *grads)`` static methods,
    invoked with ``.apply`` (python/paddle/autograd/py_layer.py)."""

    @classmethod
    def apply(cls, *args, **kwargs):
        if kwargs:
            keys = list(kwargs)

            class _KW(cls):
                @staticmethod
                def forward(ctx, *a):
                    n = len(a) - len(keys)
                    return cls.forward(ctx, *a[:n], **dict(zip(keys, a[n:])))
            out = super(PyLayer, _KW).apply(*args, *[kwargs[k] for k in keys])
        else:
            out = super().apply(*args)
        return _wrap(out)


def _wrap(o):
    if isinstance(o, torch.Tensor):
        return as_tensor(o)
    if isinstance(o, tuple):
        return tuple(_wrap(x) for x in o)
    if isinstance(o, list):
        return [_wrap(x) for x in o]
    return o


def backward(tensors, grad_tensors=None, retain_graph=False):
    tensors = [tensors] if isinstance(tensors, torch.Tensor) else list(tensors)
    if grad_tensors is not None and isinstance(grad_tensors, torch.Tensor):
        grad_tensors = [grad_tensors]
    torch.autograd.backward(tensors, grad_tensors, retain_graph=retain_graph)


def grad(outputs, inputs, grad_outputs=None, retain_graph=None, create_graph=False, only_inputs=True,
         allow_unused=False, no_grad_vars=None):
    outs = [outputs] if isinstance(outputs, torch.Tensor) else list(outputs)
    ins = [inputs] if isinstance(inputs, torch.Tensor) else list(inputs)
    if grad_outputs is not None and isinstance(grad_outputs, torch.Tensor):
        grad_outputs = [grad_outputs]
    r = torch.autograd.grad(outs, ins, grad_outputs, retain_graph=retain_graph, create_graph=create_graph,
                            allow_unused=allow_unused)
    return [None if g is None else as_tensor(g) for g in r]


class saved_tensors_hooks(torch.autograd.graph.saved_tensors_hooks):
    pass


def jacobian(ys, xs, batch_axis=None):
    if callable(ys):
        return torch.autograd.functional.jacobian(ys, xs)
    flat = ys.reshape(-1)
    rows = [torch.autograd.grad(flat[i], xs, retain_graph=True, allow_unused=True)[0].reshape(-1) for i in range(flat.numel())]
    return as_tensor(torch.stack(rows))


def hessian(ys, xs, batch_axis=None):
    if callable(ys):
        return torch.autograd.functional.hessian(ys, xs)
    g = torch.autograd.grad(ys, xs, create_graph=True)[0].reshape(-1)
    rows = [torch.autograd.grad(g[i], xs, retain_graph=True)[0].reshape(-1) for i in range(g.numel())]
    return as_tensor(torch.stack(rows))


no_grad = torch.no_grad
enable_grad = torch.enable_grad
set_grad_enabled = torch.set_grad_enabled
is_grad_enabled = torch.is_grad_enabled
