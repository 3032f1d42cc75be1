"""``paddle.nn.utils``: parameter <-> vector helpers, clip_grad_norm_, weight/spectral norm."""
from __future__ import annotations

import torch

from ..._core.tensor import as_tensor


def parameters_to_vector(parameters, name=None):
    return as_tensor(torch.cat([p.detach().reshape(-1) for p in parameters]))


def vector_to_parameters(vec, parameters, name=None):
    off = 0
    with torch.no_grad():
        for p in parameters:
            n = p.numel()
            p.copy_(vec[off:off + n].reshape(p.shape))
            off += n


def clip_grad_norm_(parameters, max_norm, norm_type=2.0, error_if_nonfinite=False):
    params = [parameters] if isinstance(parameters, torch.Tensor) else list(parameters)
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return as_tensor(torch.zeros(()))
    if norm_type == float("inf"):
        total = torch.stack([g.abs().max() for g in grads]).max()
    else:
        total = torch.stack([g.float().norm(norm_type) for g in grads]).norm(norm_type)
    if error_if_nonfinite and not torch.isfinite(total):
        raise RuntimeError("non-finite gradient norm")
    coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
    for g in grads:
        g.mul_(coef.to(g.dtype))
    return as_tensor(total)


def clip_grad_value_(parameters, clip_value):
    params = [parameters] if isinstance(parameters, torch.Tensor) else list(parameters)
    for p in params:
        if p.grad is not None:
            p.grad.clamp_(-clip_value, clip_value)


def weight_norm(layer, name="weight", dim=0):
    w = getattr(layer, name)
    from ..._core.tensor import EagerParamBase
    dims = [d for d in range(w.dim()) if d != dim]
    g = EagerParamBase(w.detach().norm(2, dims, keepdim=True))
    v = EagerParamBase(w.detach().clone())
    del layer._parameters[name]
    layer.add_parameter(name + "_g", g)
    layer.add_parameter(name + "_v", v)

    def hook(l, inputs):
        vv, gg = getattr(l, name + "_v"), getattr(l, name + "_g")
        object.__setattr__(l, name, vv * (gg / vv.norm(2, dims, keepdim=True)))
    layer._wn_hook = layer.register_forward_pre_hook(hook)
    hook(layer, None)
    return layer


def remove_weight_norm(layer, name="weight"):
    from ..._core.tensor import EagerParamBase
    w = getattr(layer, name).detach()
    layer._wn_hook.remove()
    del layer._parameters[name + "_g"], layer._parameters[name + "_v"]
    layer.__dict__.pop(name, None)
    layer.add_parameter(name, EagerParamBase(w))
    return layer


def spectral_norm(layer, name="weight", n_power_iterations=1, eps=1e-12, dim=None):
    w = getattr(layer, name)
    dim = 0 if dim is None else dim

    def hook(l, inputs):
        wv = l._parameters[name + "_orig"]
        mat = wv.movedim(dim, 0).reshape(wv.shape[dim], -1)
        u = l._sn_u
        with torch.no_grad():
            for _ in range(n_power_iterations):
                v = torch.nn.functional.normalize(mat.t() @ u, dim=0, eps=eps)
                u = torch.nn.functional.normalize(mat @ v, dim=0, eps=eps)
            l._sn_u = u
        sigma = u @ (mat @ v)
        object.__setattr__(l, name, wv / sigma)
    layer.add_parameter(name + "_orig", layer._parameters.pop(name))
    layer._sn_u = torch.nn.functional.normalize(torch.randn(w.shape[dim], device=w.device), dim=0)
    layer.register_forward_pre_hook(hook)
    hook(layer, None)
    return layer
