"""``paddle.incubate.optimizer``: LookAhead (lookahead.py:34), ModelAverage (modelaverage.py:38), LBFGS re-export."""
from __future__ import annotations

import torch

from ..._core.tensor import as_tensor


class LookAhead:
    """Every ``k`` fast steps the slow weights move ``alpha`` of the way to the fast weights and the fast weights are
    reset to them."""

    def __init__(self, inner_optimizer, alpha=0.5, k=5, name=None):
        assert inner_optimizer is not None and 0.0 <= alpha <= 1.0 and isinstance(k, int) and k > 0
        self.inner_optimizer, self.alpha, self.k = inner_optimizer, alpha, k
        self._step = 0
        self._slow = {}

    def step(self):
        self.inner_optimizer.step()
        self._step += 1
        with torch.no_grad():
            for p in self.inner_optimizer._parameter_list:
                if p.name not in self._slow:
                    self._slow[p.name] = p.detach().clone()
            if self._step % self.k == 0:
                for p in self.inner_optimizer._parameter_list:
                    slow = self._slow[p.name]
                    slow.add_(p.detach() - slow, alpha=self.alpha)
                    p.copy_(slow)

    def minimize(self, loss, startup_program=None, parameters=None, no_grad_set=None):
        """Dynamic mode: the caller ran ``loss.backward()``; apply the gradients that exist (run it when none do)."""
        has_grads = any(p.grad is not None for p in self.inner_optimizer._parameter_list)
        if not has_grads and getattr(loss, "grad_fn", None) is not None:
            loss.backward()
        self.step()
        return None, None

    def clear_grad(self, set_to_zero=True):
        self.inner_optimizer.clear_grad(set_to_zero)

    def state_dict(self):
        sd = self.inner_optimizer.state_dict()
        sd.update({f"{n}_slow_0": as_tensor(t) for n, t in self._slow.items()})
        return sd

    def __getattr__(self, item):
        return getattr(self.inner_optimizer, item)


class ModelAverage:
    """Running average of parameters over a sliding window; ``apply()`` swaps the averages in (context manager),
    ``restore()`` swaps the trained values back."""

    def __init__(self, average_window_rate, parameters=None, min_average_window=10000, max_average_window=10000, name=None):
        self.rate, self.min_w, self.max_w = average_window_rate, min_average_window, max_average_window
        self._params = list(parameters)
        self._sum = {p.name: torch.zeros_like(p.detach(), dtype=torch.float32) for p in self._params}
        self._n = 0
        self._backup = None

    def step(self):
        with torch.no_grad():
            for p in self._params:
                self._sum[p.name] += p.detach().float()
        self._n += 1
        if self._n > self.max_w:
            for k in self._sum:
                self._sum[k] *= 0.5
            self._n = self._n // 2

    def minimize(self, loss, *a, **k):
        self.step()

    def clear_grad(self, set_to_zero=True):
        """Gradients belong to the inner optimizer's parameters; cleared here for loops that drive both optimizers."""
        for p in self._params:
            if p.grad is not None:
                if set_to_zero:
                    p.grad.zero_()
                else:
                    p.grad = None

    def apply(self, executor=None, need_restore=True):
        ma = self

        class _Ctx:
            def __enter__(self_inner):
                ma._backup = {p.name: p.detach().clone() for p in ma._params}
                with torch.no_grad():
                    for p in ma._params:
                        p.copy_((ma._sum[p.name] / max(ma._n, 1)).to(p.dtype))

            def __exit__(self_inner, *exc):
                if need_restore:
                    ma.restore()
        return _Ctx()

    def restore(self, executor=None):
        if self._backup is not None:
            with torch.no_grad():
                for p in self._params:
                    p.copy_(self._backup[p.name])
            self._backup = None


from ...optimizer.extras import LBFGS  # noqa: E402,F401
from . import functional  # noqa: E402,F401


class DistributedFusedLamb:
    """LAMB whose gradients are averaged over all ranks before the update
    (python/paddle/incubate/optimizer/distributed_fused_lamb.py:121).  The reference keeps every parameter, gradient
    and moment in fused flat buffers sharded over the ranks of a node; here the update itself is
    ``paddle.optimizer.Lamb`` with fp32 master weights, preceded by one all-reduce per gradient, global-norm clipping
    before or after that all-reduce (``clip_after_allreduce``) and gradient accumulation over
    ``gradient_accumulation_steps`` calls of ``step``."""

    def __init__(self, learning_rate=0.001, lamb_weight_decay=0.01, beta1=0.9, beta2=0.999, epsilon=1e-6,
                 parameters=None, grad_clip=None, exclude_from_weight_decay_fn=None, clip_after_allreduce=True,
                 is_grad_scaled_by_nranks=True, alignment=128, use_master_param_norm=True,
                 gradient_accumulation_steps=1, use_master_acc_grad=True, nproc_per_node=None,
                 use_hierarchical_allreduce=False, name=None):
        from ...optimizer import Lamb
        self._inner = Lamb(learning_rate, lamb_weight_decay, beta1, beta2, epsilon, parameters, None,
                           exclude_from_weight_decay_fn, multi_precision=True, name=name)
        self._clip, self._clip_after = grad_clip, clip_after_allreduce
        self._scaled_by_nranks = is_grad_scaled_by_nranks
        self._acc_steps, self._acc_i = int(gradient_accumulation_steps), 0
        self._scale = None

    def __getattr__(self, name):
        return getattr(self.__dict__["_inner"], name)

    def _set_scale(self, scale):
        """Loss-scaling factor the gradients carry (divided out before the update)."""
        self._scale = scale

    def _params_with_grad(self):
        return [p for p in self._inner._parameter_list if getattr(p, "grad", None) is not None]

    def _apply_clip(self, params):
        if self._clip is not None:
            for (p, g) in self._clip([(p, p.grad) for p in params]):
                if g is not p.grad:
                    p.grad.copy_(g)

    def step(self):
        from ...distributed import collective as C
        self._acc_i += 1
        if self._acc_i % self._acc_steps != 0:
            return                                       # gradients keep accumulating in .grad
        params = self._params_with_grad()
        world = C.get_world_size() if C.is_initialized() else 1
        if self._scale is not None:
            for p in params:
                p.grad.div_(float(self._scale))
        if not self._clip_after:
            self._apply_clip(params)
        if world > 1:
            for p in params:
                C.all_reduce(p.grad)
                if not self._scaled_by_nranks:
                    p.grad.div_(world)
        if self._acc_steps > 1:
            for p in params:
                p.grad.div_(self._acc_steps)
        if self._clip_after:
            self._apply_clip(params)
        self._inner.step()

    def clear_grad(self, set_to_zero=True):
        if self._acc_i % self._acc_steps == 0:
            self._inner.clear_grad(set_to_zero)

    def minimize(self, loss, startup_program=None, parameters=None, no_grad_set=None):
        loss.backward()
        self.step()
        self.clear_grad()
