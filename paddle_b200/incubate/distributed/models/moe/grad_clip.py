"""Global-norm clipping aware of expert parameters (python/paddle/incubate/distributed/models/moe/grad_clip.py:28):
the squared norm of expert parameters (``is_moe_param(p)``) is summed over the expert-parallel group before it is
combined with the norm of the replicated parameters."""
from __future__ import annotations

import torch

from .....distributed import collective as C
from .....nn.clip import ClipGradByGlobalNorm


class ClipGradForMOEByGlobalNorm(ClipGradByGlobalNorm):
    def __init__(self, clip_norm, is_expert_param_func=None, moe_group=None, group_name="default_moe_group"):
        super().__init__(clip_norm)
        self.is_expert = is_expert_param_func or (lambda p: getattr(p, "is_moe_param", False) or getattr(p, "no_sync", False))
        self.moe_group = moe_group

    def _sq(self, grads):
        return sum((g.float() ** 2).sum() for g in grads) if grads else None

    def __call__(self, params_grads):
        normal = [g for p, g in params_grads if g is not None and getattr(p, "need_clip", True) and not self.is_expert(p)]
        expert = [g for p, g in params_grads if g is not None and getattr(p, "need_clip", True) and self.is_expert(p)]
        sq_n, sq_e = self._sq(normal), self._sq(expert)
        if sq_e is not None and self.moe_group is not None and self.moe_group.nranks > 1:
            sq_e = sq_e.clone()
            C.all_reduce(sq_e, group=self.moe_group)
        total = (sq_n if sq_n is not None else 0.0) + (sq_e if sq_e is not None else 0.0)
        if not isinstance(total, torch.Tensor):
            return params_grads
        norm = total.sqrt()
        coef = self.clip_norm / torch.clamp(norm, min=self.clip_norm)
        out = []
        for p, g in params_grads:
            if g is not None and getattr(p, "need_clip", True):
                g = g * coef.to(g.dtype)
            out.append((p, g))
        return out
