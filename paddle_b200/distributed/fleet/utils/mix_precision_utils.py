"""fp32 gradient accumulation for low-precision parameters (``main_grad``).

Mirrors python/paddle/distributed/fleet/utils/mix_precision_utils.py: ``MixPrecisionLayer`` (:35-95)
gives every parameter an fp32 ``main_grad`` that backward accumulates into, ``MixPrecisionOptimizer``
(:97-195) makes the inner optimizer read ``main_grad``.  Here the weight-gradient GEMM, the RMSNorm
backward and the embedding backward add straight into ``main_grad`` from their epilogues; any gradient
that still arrives as a low-precision ``.grad`` is folded in by a post-accumulate hook and dropped.
"""
from __future__ import annotations

import torch

from ...._core.tensor import as_tensor


def _fold_grad_hook(p):
    g = torch.Tensor.grad.__get__(p)
    if g is None:
        return
    mg = p.main_grad
    if g.is_cuda and g.dtype == torch.bfloat16 and g.is_contiguous():
        from ....ops import native
        native.accumulate_into_f32(g, mg)
    else:
        mg.add_(g.to(torch.float32))
    torch.Tensor.grad.__set__(p, None)
    hook = getattr(p, "_main_grad_ready_hook", None)
    if hook is not None:
        hook(p)


def enable_main_grad(layer):
    """Allocate a persistent fp32 ``main_grad`` for every trainable parameter of ``layer``."""
    for p in layer.parameters():
        if not p.requires_grad or getattr(p, "main_grad", None) is not None:
            continue
        p.main_grad = as_tensor(torch.zeros(p.shape, dtype=torch.float32, device=p.device))
        p._main_grad_persistent = True
        p._main_grad_hook_handle = p.register_post_accumulate_grad_hook(_fold_grad_hook)
    return layer


class MixPrecisionLayer:
    """Wrapper with the reference's constructor; attribute access is forwarded to the wrapped layer."""

    def __init__(self, layers, dtype="float16"):
        self.__dict__["_layers"] = layers
        self.__dict__["_dtype"] = dtype
        enable_main_grad(layers)

    def __call__(self, *inputs, **kwargs):
        return self._layers(*inputs, **kwargs)

    forward = __call__

    def __getattr__(self, name):
        return getattr(self.__dict__["_layers"], name)

    def __setattr__(self, name, value):
        setattr(self.__dict__["_layers"], name, value)

    def state_dict(self, *a, **k):
        return self._layers.state_dict(*a, **k)

    def set_state_dict(self, *a, **k):
        return self._layers.set_state_dict(*a, **k)


class MixPrecisionOptimizer:
    """The optimizers of this framework already prefer ``main_grad``; the wrapper only forwards."""

    def __init__(self, optimizer):
        self._inner_opt = optimizer

    def __getattr__(self, name):
        return getattr(self._inner_opt, name)

    def step(self):
        return self._inner_opt.step()

    def clear_grad(self, set_to_zero=True):
        return self._inner_opt.clear_grad(set_to_zero)


def unscale_method(self, optimizer):
    return self.unscale_(optimizer)


class MixPrecisionScaler:
    def __init__(self, scaler):
        self._inner = scaler

    def __getattr__(self, name):
        return getattr(self._inner, name)
