"""Gradient clipping (python/paddle/nn/clip.py).  Clip objects are callables on a list of
``(param, grad)`` pairs, as the optimizers expect; ``ClipGradByGlobalNorm`` computes the squared
norms with one multi-tensor kernel on GPU."""
from __future__ import annotations

import torch


class ClipGradBase:
    def __call__(self, params_grads):
        return self._dygraph_clip(params_grads)


class ClipGradByValue(ClipGradBase):
    def __init__(self, max, min=None):
        self.max = float(max)
        self.min = -self.max if min is None else float(min)

    def _dygraph_clip(self, params_grads):
        out = []
        for p, g in params_grads:
            if g is None or not getattr(p, "need_clip", True):
                out.append((p, g))
            else:
                out.append((p, g.clamp(self.min, self.max)))
        return out


class ClipGradByNorm(ClipGradBase):
    def __init__(self, clip_norm):
        self.clip_norm = float(clip_norm)

    def _dygraph_clip(self, params_grads):
        out = []
        for p, g in params_grads:
            if g is None or not getattr(p, "need_clip", True):
                out.append((p, g))
                continue
            n = g.float().norm()
            out.append((p, (g * (self.clip_norm / torch.maximum(n, torch.tensor(self.clip_norm, device=g.device)))).to(g.dtype)))
        return out


class ClipGradByGlobalNorm(ClipGradBase):
    """g *= clip_norm / max(global_norm, clip_norm) (python/paddle/nn/clip.py ``ClipGradByGlobalNorm``)."""

    def __init__(self, clip_norm, group_name="default_group", auto_skip_clip=False):
        self.clip_norm = float(clip_norm)
        self.group_name = group_name
        self.auto_skip_clip = auto_skip_clip
        self._table = None

    def global_norm_sq(self, grads):
        """Sum of squares over `grads` as a 1-element fp32 tensor."""
        grads = [g for g in grads if g is not None]
        if not grads:
            return None
        if grads[0].is_cuda and all(g.is_contiguous() and g.dtype in (torch.float32, torch.bfloat16) for g in grads):
            from ..ops import native
            if self._table is None or not self._table.matches(grads, grads):
                self._table = native.TensorTable(grads, grads)
            return self._table.sq_l2_norm()
        return torch.stack([g.float().pow(2).sum() for g in grads]).sum().reshape(1)

    def clip_coef(self, norm_sq):
        gn = norm_sq.sqrt()
        return self.clip_norm / torch.maximum(gn, torch.full_like(gn, self.clip_norm))

    def _dygraph_clip(self, params_grads):
        grads = [g for p, g in params_grads if g is not None and getattr(p, "need_clip", True)]
        if not grads:
            return params_grads
        coef = self.clip_coef(self.global_norm_sq(grads))
        out = []
        for p, g in params_grads:
            if g is None or not getattr(p, "need_clip", True):
                out.append((p, g))
            else:
                out.append((p, g.mul_(coef.to(g.dtype))))
        return out


def clip_by_norm(x, max_norm, name=None):
    """``x * max_norm / max(norm(x), max_norm)`` (python/paddle/nn/clip.py ``clip_by_norm``)."""
    t = x.as_subclass(torch.Tensor)
    norm = torch.linalg.vector_norm(t.float())
    scale = float(max_norm) / torch.clamp(norm, min=float(max_norm))
    from .._core.tensor import as_tensor
    return as_tensor((t.float() * scale).to(t.dtype))


def merge_selected_rows(x, name=None):
    """Sums duplicate rows of a row-sparse gradient.  Row-sparse gradients are sparse COO tensors here."""
    return x.coalesce() if getattr(x, "is_sparse", False) else x


def get_tensor_from_selected_rows(x, name=None):
    return x.coalesce().values() if getattr(x, "is_sparse", False) else x


_legacy_clip = {"clip": None}


def set_gradient_clip(clip, param_list=None, program=None):
    """Legacy global setting read by optimizers created without ``grad_clip`` (deprecated in the reference)."""
    import warnings
    warnings.warn("set_gradient_clip is deprecated: pass grad_clip to the optimizer instead")
    _legacy_clip["clip"] = clip
    if param_list is not None:
        for p in param_list:
            p.gradient_clip_attr = clip


class ErrorClipByValue:
    """Clips the gradient flowing INTO a variable (legacy static-graph attribute)."""

    def __init__(self, max, min=None):
        self.max = float(max)
        self.min = float(min) if min is not None else -self.max


BaseErrorClipAttr = ErrorClipByValue


def error_clip_callback(block, context):
    pass


def append_gradient_clip_ops(param_grads):
    clip = _legacy_clip["clip"]
    return clip(param_grads) if clip is not None else param_grads
