"""Decomposition rules: composite operator -> primitive operators (python/paddle/decomposition/rules.py; the bulk of
the reference's rules are the C++ templates of paddle/fluid/primitive/composite/composite.h: softmax, gelu, layer_norm,
rms_norm, silu, ... - the same set is covered here).  A rule takes the arguments of the recorded call it replaces (the
torch-level signature the static-graph recorder saw) and uses only operators of :data:`primitives.PRIMITIVES`.
Reductions and normalisations compute in fp32 and cast back, as the reference's rules do for fp16 / bf16 inputs."""
from __future__ import annotations

import math

import torch

from .register import register_decomp


def _f32(x):
    return (x.float(), x.dtype) if x.dtype in (torch.bfloat16, torch.float16) else (x, None)


def _back(y, dt):
    return y.to(dt) if dt is not None else y


def _dim(args, kwargs, pos=1, default=-1):
    if "dim" in kwargs:
        return kwargs["dim"]
    if "axis" in kwargs:
        return kwargs["axis"]
    return args[pos - 1] if len(args) >= pos and args[pos - 1] is not None else default


# ------------------------------------------------------------------------------------------------ activations
@register_decomp("pd_op.relu")
def relu(x, inplace=False):
    return torch.maximum(x, torch.zeros_like(x))


@register_decomp("pd_op.relu6")
def relu6(x, inplace=False):
    return torch.minimum(torch.maximum(x, torch.zeros_like(x)), torch.full_like(x, 6.0))


@register_decomp("pd_op.leaky_relu")
def leaky_relu(x, negative_slope=0.01, inplace=False):
    return torch.where(x > 0, x, x * negative_slope)


@register_decomp("pd_op.sigmoid")
def sigmoid(x):
    xf, dt = _f32(x)
    return _back(1.0 / (1.0 + torch.exp(-xf)), dt)


@register_decomp("pd_op.silu")
def silu(x, inplace=False):
    xf, dt = _f32(x)
    return _back(xf / (1.0 + torch.exp(-xf)), dt)


@register_decomp("pd_op.gelu")
def gelu(x, approximate="none"):
    xf, dt = _f32(x)
    if approximate == "tanh":
        y = 0.5 * xf * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (xf + 0.044715 * xf * xf * xf)))
    else:
        y = 0.5 * xf * (1.0 + torch.erf(xf * (1.0 / math.sqrt(2.0))))
    return _back(y, dt)


@register_decomp("pd_op.hardswish")
def hardswish(x, inplace=False):
    return x * torch.minimum(torch.maximum(x + 3.0, torch.zeros_like(x)), torch.full_like(x, 6.0)) / 6.0


@register_decomp("pd_op.hardsigmoid")
def hardsigmoid(x, inplace=False):
    return torch.minimum(torch.maximum(x / 6.0 + 0.5, torch.zeros_like(x)), torch.ones_like(x))


@register_decomp("pd_op.hardtanh")
def hardtanh(x, min_val=-1.0, max_val=1.0, inplace=False):
    return torch.minimum(torch.maximum(x, torch.full_like(x, min_val)), torch.full_like(x, max_val))


@register_decomp("pd_op.softplus")
def softplus(x, beta=1.0, threshold=20.0):
    xf, dt = _f32(x)
    soft = torch.log(1.0 + torch.exp(xf * beta)) / beta
    return _back(torch.where(xf * beta > threshold, xf, soft), dt)


@register_decomp("pd_op.softsign")
def softsign(x):
    return x / (1.0 + torch.abs(x))


@register_decomp("pd_op.mish")
def mish(x, inplace=False):
    xf, dt = _f32(x)
    return _back(xf * torch.tanh(torch.log(1.0 + torch.exp(xf))), dt)


@register_decomp("pd_op.elu")
def elu(x, alpha=1.0, inplace=False):
    return torch.where(x > 0, x, alpha * (torch.exp(x) - 1.0))


@register_decomp("pd_op.selu")
def selu(x, inplace=False):
    alpha, scale = 1.6732632423543772, 1.0507009873554805
    return scale * torch.where(x > 0, x, alpha * (torch.exp(x) - 1.0))


@register_decomp("pd_op.swiglu")
def swiglu(x, y=None):
    if y is None:
        x, y = torch.chunk(x, 2, -1)
    xf, dt = _f32(x)
    return _back(xf / (1.0 + torch.exp(-xf)) * (y.float() if dt is not None else y), dt)


# ------------------------------------------------------------------------------------------------ softmax family
@register_decomp("pd_op.softmax")
def softmax(x, *args, **kwargs):
    dim = _dim(args, kwargs)
    xf, dt = _f32(x)
    if kwargs.get("dtype") is not None:
        xf, dt = x.to(kwargs["dtype"]), None
    e = torch.exp(xf - torch.amax(xf, dim, keepdim=True))
    return _back(e / torch.sum(e, dim, keepdim=True), dt)


@register_decomp("pd_op.log_softmax")
def log_softmax(x, *args, **kwargs):
    dim = _dim(args, kwargs)
    xf, dt = _f32(x)
    if kwargs.get("dtype") is not None:
        xf, dt = x.to(kwargs["dtype"]), None
    sh = xf - torch.amax(xf, dim, keepdim=True)
    return _back(sh - torch.log(torch.sum(torch.exp(sh), dim, keepdim=True)), dt)


@register_decomp("pd_op.logsumexp")
def logsumexp(x, dim, keepdim=False):
    xf, dt = _f32(x)
    m = torch.amax(xf, dim, keepdim=True)
    out = torch.log(torch.sum(torch.exp(xf - m), dim, keepdim=True)) + m
    if not keepdim:
        out = torch.squeeze(out, dim)
    return _back(out, dt)


# ------------------------------------------------------------------------------------------------ normalisation
@register_decomp("pd_op.layer_norm")
def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    dims = tuple(range(x.dim() - len(tuple(normalized_shape)), x.dim()))
    xf, dt = _f32(x)
    mean = torch.mean(xf, dims, keepdim=True)
    cen = xf - mean
    var = torch.mean(cen * cen, dims, keepdim=True)
    y = cen * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * (weight.float() if dt is not None else weight)
    if bias is not None:
        y = y + (bias.float() if dt is not None else bias)
    return _back(y, dt)


@register_decomp("pd_op.rms_norm")
def rms_norm(x, normalized_shape, weight=None, eps=None):
    dims = tuple(range(x.dim() - len(tuple(normalized_shape)), x.dim()))
    xf, dt = _f32(x)
    eps = torch.finfo(x.dtype).eps if eps is None else eps
    y = xf * torch.rsqrt(torch.mean(xf * xf, dims, keepdim=True) + eps)
    if weight is not None:
        y = y * (weight.float() if dt is not None else weight)
    return _back(y, dt)


@register_decomp("pd_op.batch_norm")
def batch_norm(x, running_mean, running_var, weight=None, bias=None, training=False, momentum=0.1, eps=1e-5):
    """Inference form (running statistics); the training form updates buffers in place and stays composite."""
    if training:
        return torch.nn.functional.batch_norm(x, running_mean, running_var, weight, bias, True, momentum, eps)
    shape = [1, -1] + [1] * (x.dim() - 2)
    y = (x - torch.reshape(running_mean, shape)) * torch.rsqrt(torch.reshape(running_var, shape) + eps)
    if weight is not None:
        y = y * torch.reshape(weight, shape)
    if bias is not None:
        y = y + torch.reshape(bias, shape)
    return y


@register_decomp("pd_op.group_norm")
def group_norm(x, num_groups, weight=None, bias=None, eps=1e-5):
    n, c = x.shape[0], x.shape[1]
    xf, dt = _f32(x)
    g = torch.reshape(xf, (n, num_groups, -1))
    mean = torch.mean(g, 2, keepdim=True)
    cen = g - mean
    var = torch.mean(cen * cen, 2, keepdim=True)
    y = torch.reshape(cen * torch.rsqrt(var + eps), x.shape)
    shape = [1, c] + [1] * (x.dim() - 2)
    if weight is not None:
        y = y * torch.reshape(weight.float() if dt is not None else weight, shape)
    if bias is not None:
        y = y + torch.reshape(bias.float() if dt is not None else bias, shape)
    return _back(y, dt)


@register_decomp("pd_op.instance_norm")
def instance_norm(x, running_mean=None, running_var=None, weight=None, bias=None, use_input_stats=True, momentum=0.1,
                  eps=1e-5):
    dims = tuple(range(2, x.dim()))
    mean = torch.mean(x, dims, keepdim=True)
    cen = x - mean
    y = cen * torch.rsqrt(torch.mean(cen * cen, dims, keepdim=True) + eps)
    shape = [1, -1] + [1] * (x.dim() - 2)
    if weight is not None:
        y = y * torch.reshape(weight, shape)
    if bias is not None:
        y = y + torch.reshape(bias, shape)
    return y


@register_decomp("pd_op.normalize")
def normalize(x, p=2.0, dim=1, eps=1e-12, out=None):
    norm = torch.pow(torch.sum(torch.pow(torch.abs(x), p), dim, keepdim=True), 1.0 / p)
    return x / torch.maximum(norm, torch.full_like(norm, eps))


# ------------------------------------------------------------------------------------------------ statistics
@register_decomp("pd_op.var")
def var(x, dim=None, *, correction=1, keepdim=False, unbiased=None):
    if unbiased is not None:
        correction = 1 if unbiased else 0
    dims = tuple(range(x.dim())) if dim is None else ((dim,) if isinstance(dim, int) else tuple(dim))
    n = 1
    for d in dims:
        n *= x.shape[d]
    cen = x - torch.mean(x, dims, keepdim=True)
    return torch.sum(cen * cen, dims, keepdim=keepdim) / max(n - correction, 0)


@register_decomp("pd_op.std")
def std(x, dim=None, *, correction=1, keepdim=False, unbiased=None):
    return torch.sqrt(var(x, dim, correction=correction, keepdim=keepdim, unbiased=unbiased))


@register_decomp("pd_op.square")
def square(x):
    return x * x


@register_decomp("pd_op.squared_l2_norm")
def squared_l2_norm(x):
    xf, _ = _f32(x)
    return torch.reshape(torch.sum(xf * xf), (1,))


# ------------------------------------------------------------------------------------------------ linear algebra
@register_decomp("pd_op.linear")
def linear(x, weight, bias=None):
    """torch layout: weight [out, in]."""
    y = torch.matmul(x, torch.transpose(weight, -1, -2))
    return y if bias is None else y + bias


@register_decomp("pd_op.addmm")
def addmm(inp, mat1, mat2, *, beta=1, alpha=1):
    return beta * inp + alpha * torch.matmul(mat1, mat2)


@register_decomp("pd_op.baddbmm")
def baddbmm(inp, b1, b2, *, beta=1, alpha=1):
    return beta * inp + alpha * torch.matmul(b1, b2)


@register_decomp("pd_op.addcmul")
def addcmul(inp, t1, t2, *, value=1):
    return inp + value * t1 * t2


@register_decomp("pd_op.addcdiv")
def addcdiv(inp, t1, t2, *, value=1):
    return inp + value * t1 / t2


@register_decomp("pd_op.lerp")
def lerp(start, end, weight):
    return start + weight * (end - start)


# ------------------------------------------------------------------------------------------------ losses / misc
@register_decomp("pd_op.dropout")
def dropout(x, p=0.5, training=True, inplace=False):
    if not training or p == 0.0:
        return x
    keep = (torch.rand_like(x, dtype=torch.float32) >= p).to(x.dtype)
    return x * keep / (1.0 - p)


@register_decomp("pd_op.mse_loss")
def mse_loss(x, target, size_average=None, reduce=None, reduction="mean", weight=None):
    d = (x - target) * (x - target)
    return torch.mean(d) if reduction == "mean" else (torch.sum(d) if reduction == "sum" else d)


@register_decomp("pd_op.l1_loss")
def l1_loss(x, target, size_average=None, reduce=None, reduction="mean"):
    d = torch.abs(x - target)
    return torch.mean(d) if reduction == "mean" else (torch.sum(d) if reduction == "sum" else d)


@register_decomp("pd_op.smooth_l1_loss")
def smooth_l1_loss(x, target, size_average=None, reduce=None, reduction="mean", beta=1.0):
    d = torch.abs(x - target)
    v = torch.where(d < beta, 0.5 * d * d / beta, d - 0.5 * beta)
    return torch.mean(v) if reduction == "mean" else (torch.sum(v) if reduction == "sum" else v)


@register_decomp("pd_op.binary_cross_entropy_with_logits")
def binary_cross_entropy_with_logits(x, target, weight=None, size_average=None, reduce=None, reduction="mean",
                                     pos_weight=None):
    # max(x, 0) - x t + log(1 + exp(-|x|)), with the positive-class weight folded in
    lw = 1.0 if pos_weight is None else 1.0 + (pos_weight - 1.0) * target
    v = (1.0 - target) * x + lw * (torch.log(1.0 + torch.exp(-torch.abs(x))) + torch.maximum(-x, torch.zeros_like(x)))
    if weight is not None:
        v = v * weight
    return torch.mean(v) if reduction == "mean" else (torch.sum(v) if reduction == "sum" else v)


@register_decomp("pd_op.cross_entropy")
def cross_entropy(x, target, weight=None, size_average=None, ignore_index=-100, reduce=None, reduction="mean",
                  label_smoothing=0.0):
    """Class-index targets over the last axis of a 2-D input (the softmax-with-cross-entropy case)."""
    if x.dim() != 2 or target.dtype not in (torch.int64, torch.int32) or weight is not None or label_smoothing:
        return torch.nn.functional.cross_entropy(x, target, weight, size_average, ignore_index, reduce, reduction,
                                                 label_smoothing)
    xf, _ = _f32(x)
    sh = xf - torch.amax(xf, 1, keepdim=True)
    lse = torch.log(torch.sum(torch.exp(sh), 1))
    valid = target != ignore_index
    safe = torch.where(valid, target, torch.zeros_like(target)).to(torch.int64)
    picked = torch.squeeze(torch.gather(sh, 1, torch.unsqueeze(safe, 1)), 1)
    loss = torch.where(valid, lse - picked, torch.zeros_like(lse))
    if reduction == "mean":
        return torch.sum(loss) / torch.sum(valid.to(loss.dtype))
    return torch.sum(loss) if reduction == "sum" else loss
