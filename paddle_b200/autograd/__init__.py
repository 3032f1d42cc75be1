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
    """Backward from several tensors at once; a missing (or ``None``) initial gradient is ones of the tensor's shape."""
    tensors = [tensors] if isinstance(tensors, torch.Tensor) else list(tensors)
    if grad_tensors is None:
        grad_tensors = [None] * len(tensors)
    elif isinstance(grad_tensors, torch.Tensor):
        grad_tensors = [grad_tensors]
    grad_tensors = list(grad_tensors)
    if len(grad_tensors) != len(tensors):
        raise ValueError("The length of grad_tensors must be equal to tensors")
    grads = [torch.ones_like(t.detach().as_subclass(torch.Tensor)) if g is None else g for t, g in zip(tensors, grad_tensors)]
    torch.autograd.backward(tensors, grads, retain_graph=retain_graph)


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


def _jac_one(y, x, batch_axis, create_graph=False):
    """d y / d x as [M, N] (``batch_axis=None``) or [B, M, N] (``batch_axis=0``: sample b of y depends on sample b of x
    only); inputs y does not depend on give zeros."""
    if batch_axis is None:
        flat = y.reshape(-1)
        rows = []
        for i in range(flat.numel()):
            g = torch.autograd.grad(flat[i], x, retain_graph=True, create_graph=create_graph, allow_unused=True)[0]
            rows.append(torch.zeros_like(x).reshape(-1) if g is None else g.reshape(-1))
        return torch.stack(rows) if rows else x.new_zeros(0, x.numel())
    if batch_axis != 0:
        raise ValueError("batch_axis should be None or 0")
    B = y.shape[0]
    yf = y.reshape(B, -1)
    cols = []
    for m in range(yf.shape[1]):
        g = torch.autograd.grad(yf[:, m].sum(), x, retain_graph=True, create_graph=create_graph, allow_unused=True)[0]
        cols.append(torch.zeros_like(x).reshape(B, -1) if g is None else g.reshape(B, -1))
    return torch.stack(cols, 1)


def jacobian(ys, xs, batch_axis=None):
    """Jacobian of ``ys`` with respect to ``xs`` (python/paddle/autograd/autograd.py ``jacobian``): a tensor for tensor
    arguments, a tuple over ``xs`` (nested in a tuple over ``ys``) when either is a sequence; flattened to [M, N], or
    [B, M, N] with ``batch_axis=0``.  A callable ``ys`` is evaluated at ``xs`` first."""
    if callable(ys):
        args = xs if isinstance(xs, (list, tuple)) else (xs,)
        ys = ys(*args)
    many_y, many_x = isinstance(ys, (list, tuple)), isinstance(xs, (list, tuple))
    out = tuple(tuple(as_tensor(_jac_one(y, x, batch_axis)) for x in (xs if many_x else [xs])) for y in (ys if many_y else [ys]))
    if not many_x:
        out = tuple(r[0] for r in out)
    return out if many_y else out[0]


def hessian(ys, xs, batch_axis=None):
    """Second derivatives of a scalar ``ys`` (one scalar per sample with ``batch_axis=0``): [N, N] for one input, a
    tuple of tuples ``H[i][j] = d2 y / d x_i d x_j`` for several."""
    if callable(ys):
        args = xs if isinstance(xs, (list, tuple)) else (xs,)
        ys = ys(*args)
    many_x = isinstance(xs, (list, tuple))
    xlist = list(xs) if many_x else [xs]
    if batch_axis is None and ys.numel() != 1:
        raise ValueError("hessian needs a scalar ys (or batch_axis=0 with one scalar per sample)")
    firsts = []
    for x in xlist:
        target = ys.sum() if batch_axis == 0 else ys.reshape(())
        g = torch.autograd.grad(target, x, create_graph=True, allow_unused=True)[0]
        firsts.append(torch.zeros_like(x) if g is None else g)
    rows = []
    for gi, xi in zip(firsts, xlist):
        row = []
        for xj in xlist:
            if not gi.requires_grad:
                n_i = xi.numel() if batch_axis is None else xi[0].numel()
                n_j = xj.numel() if batch_axis is None else xj[0].numel()
                row.append(as_tensor(xi.new_zeros((n_i, n_j) if batch_axis is None else (xi.shape[0], n_i, n_j))))
            else:
                row.append(as_tensor(_jac_one(gi if batch_axis is None else gi.reshape(gi.shape[0], -1), xj, batch_axis)))
        rows.append(tuple(row))
    return tuple(rows) if many_x else rows[0][0]


no_grad = torch.no_grad
enable_grad = torch.enable_grad
set_grad_enabled = torch.set_grad_enabled
is_grad_enabled = torch.is_grad_enabled
