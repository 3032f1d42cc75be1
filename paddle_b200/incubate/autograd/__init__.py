"""``paddle.incubate.autograd`` (python/paddle/incubate/autograd/): functional differentiation helpers.
``vjp`` / ``jvp`` / ``Jacobian`` / ``Hessian`` evaluate a function and differentiate it with the eager engine
(forward mode uses the double-backward trick); ``enable_prim`` toggles a flag only, because operators are never
decomposed into primitives here."""
from __future__ import annotations

import torch

from ..._core.tensor import as_tensor

_prim = False


def enable_prim():
    global _prim
    _prim = True


def disable_prim():
    global _prim
    _prim = False


def prim_enabled():
    return _prim


def _seq(x):
    return list(x) if isinstance(x, (list, tuple)) else [x]


def _p(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


def _pack(vals, like):
    out = [as_tensor(v) for v in vals]
    return out if isinstance(like, (list, tuple)) else out[0]


def vjp(func, xs, v=None):
    xs_l = [_p(x).detach().requires_grad_(True) for x in _seq(xs)]
    ys = func(*[as_tensor(x) for x in xs_l])
    ys_l = [_p(y) for y in _seq(ys)]
    vs = [torch.ones_like(y) for y in ys_l] if v is None else [_p(t) for t in _seq(v)]
    grads = torch.autograd.grad(ys_l, xs_l, vs, allow_unused=True)
    grads = [torch.zeros_like(x) if g is None else g for g, x in zip(grads, xs_l)]
    return ys, _pack(grads, xs)


def jvp(func, xs, v=None):
    xs_l = [_p(x).detach().requires_grad_(True) for x in _seq(xs)]
    ys = func(*[as_tensor(x) for x in xs_l])
    ys_l = [_p(y) for y in _seq(ys)]
    vs = [torch.ones_like(x) for x in xs_l] if v is None else [_p(t) for t in _seq(v)]
    us = [torch.zeros_like(y, requires_grad=True) for y in ys_l]
    g = torch.autograd.grad(ys_l, xs_l, us, create_graph=True, allow_unused=True)
    g = [torch.zeros_like(x) if gi is None else gi for gi, x in zip(g, xs_l)]
    out = torch.autograd.grad(g, us, vs, allow_unused=True)
    out = [torch.zeros_like(y) if o is None else o for o, y in zip(out, ys_l)]
    return ys, _pack(out, ys)


def forward_grad(outputs, inputs, grad_inputs=None):
    raise RuntimeError("forward_grad works on static programs lowered to primitive operators, which this framework "
                       "does not have; use incubate.autograd.jvp")


def grad(outputs, inputs, grad_outputs=None):
    from ... import autograd as _ag
    return _ag.grad(outputs, inputs, grad_outputs, allow_unused=True) if hasattr(_ag, "grad") else None


class Jacobian:
    """Lazily evaluated Jacobian of ``func`` at ``xs``; rows are outputs, columns inputs (both flattened; with
    ``is_batched`` the leading dimension is kept).  Index it (``J[:]``, ``J[0, 1]``) to get values."""

    def __init__(self, func, xs, is_batched=False):
        self._batched = is_batched
        xs_l = [_p(x).detach() for x in _seq(xs)]

        def flat_fn(*a):
            ys = func(*[as_tensor(t) for t in a])
            ys_l = [_p(y) for y in _seq(ys)]
            if is_batched:
                return torch.cat([y.reshape(y.shape[0], -1) for y in ys_l], -1)
            return torch.cat([y.reshape(-1) for y in ys_l])
        jac = torch.autograd.functional.jacobian(flat_fn, tuple(xs_l), vectorize=False, create_graph=False)
        if is_batched:
            # d y[b, i] / d x[b, j]: take the diagonal over the two batch dimensions
            parts = []
            for j, x in zip(jac, xs_l):
                B = x.shape[0]
                j = j.reshape(B, j.shape[1], B, -1)
                parts.append(torch.stack([j[b, :, b] for b in range(B)]))
            self._mat = torch.cat(parts, -1)
        else:
            self._mat = torch.cat([j.reshape(j.shape[0], -1) for j in jac], -1)

    @property
    def shape(self):
        return list(self._mat.shape)

    def __getitem__(self, idx):
        return as_tensor(self._mat[idx])


class Hessian(Jacobian):
    def __init__(self, func, xs, is_batched=False):
        def grad_fn(*a):
            xs_l = [_p(t) for t in a]
            with torch.enable_grad():
                xs_r = [t.detach().requires_grad_(True) if not t.requires_grad else t for t in xs_l]
                y = _p(func(*[as_tensor(t) for t in xs_r]))
                g = torch.autograd.grad(y.sum(), xs_r, create_graph=True)
            if is_batched:
                return as_tensor(torch.cat([gi.reshape(gi.shape[0], -1) for gi in g], -1))
            return as_tensor(torch.cat([gi.reshape(-1) for gi in g]))
        self._batched = is_batched
        xs_l = [_p(x).detach() for x in _seq(xs)]

        def flat(*a):
            return _p(grad_fn(*a))
        jac = torch.autograd.functional.jacobian(flat, tuple(xs_l), vectorize=False, create_graph=False)
        if is_batched:
            parts = []
            for j, x in zip(jac, xs_l):
                B = x.shape[0]
                j = j.reshape(B, j.shape[1], B, -1)
                parts.append(torch.stack([j[b, :, b] for b in range(B)]))
            self._mat = torch.cat(parts, -1)
        else:
            self._mat = torch.cat([j.reshape(j.shape[0], -1) for j in jac], -1)


from ..._core.submodule_alias import alias_submodules as _alias  # noqa: E402
_alias(__name__, ("functional", "primapi", "utils"))
