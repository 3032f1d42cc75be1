"""ASGD, RAdam, NAdam, Rprop and LBFGS (python/paddle/optimizer/{asgd,radam,nadam,rprop,lbfgs}.py)."""
from __future__ import annotations

import torch

from .optimizer import L2Decay, Optimizer
from .sgd import _TorchBacked


class RAdam(_TorchBacked):
    _cls = torch.optim.RAdam

    def __init__(self, learning_rate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8, parameters=None, weight_decay=None,
                 grad_clip=None, name=None):
        super().__init__(learning_rate, parameters, weight_decay, grad_clip, name, betas=(beta1, beta2), eps=epsilon)


class NAdam(_TorchBacked):
    _cls = torch.optim.NAdam

    def __init__(self, learning_rate=0.002, beta1=0.9, beta2=0.999, epsilon=1e-8, momentum_decay=0.004,
                 parameters=None, weight_decay=None, grad_clip=None, name=None):
        super().__init__(learning_rate, parameters, weight_decay, grad_clip, name, betas=(beta1, beta2), eps=epsilon,
                         momentum_decay=momentum_decay)


class Rprop(Optimizer):
    """Sign-based resilient propagation: per-element step sizes grow by ``etas[1]`` while the gradient keeps its sign
    and shrink by ``etas[0]`` when it flips (the flipped element skips one update)."""

    def __init__(self, learning_rate=0.001, learning_rate_range=(1e-5, 50), parameters=None, etas=(0.5, 1.2),
                 grad_clip=None, multi_precision=False, name=None):
        if not 0.0 < learning_rate_range[0] <= learning_rate <= learning_rate_range[1]:
            raise ValueError("'0.0 < learning_rate_range[0] <= learning_rate <= learning_rate_range[1]' must be true")
        if not 0.0 < etas[0] < 1.0 < etas[1]:
            raise ValueError("'0.0 < etas[0] < 1.0 < etas[1]' must be true")
        super().__init__(learning_rate, parameters, None, grad_clip, name, multi_precision)
        self._range, self._etas = learning_rate_range, etas
        self._state = {}

    def _apply(self, pgs, grad_scale):
        lo, hi = self._range
        dn, up = self._etas
        for p, g, _ in pgs:
            w = p.as_subclass(torch.Tensor)
            g = g.as_subclass(torch.Tensor).to(w.dtype)
            st = self._state.get(p.name)
            if st is None:
                st = self._state[p.name] = {"prev": torch.zeros_like(w), "lr": torch.full_like(w, self.get_lr())}
            sign = (g * st["prev"]).sign()
            st["lr"] = torch.where(sign > 0, st["lr"] * up, torch.where(sign < 0, st["lr"] * dn, st["lr"])).clamp_(lo, hi)
            g = torch.where(sign < 0, torch.zeros_like(g), g)
            w.sub_(st["lr"] * g.sign())
            st["prev"] = g


class ASGD(Optimizer):
    """Stochastic average gradient: keeps the last ``batch_num`` gradients ``y_i`` and their running sum ``d`` and
    steps along ``d / min(m + 1, batch_num)``."""

    def __init__(self, learning_rate=0.001, batch_num=1, parameters=None, weight_decay=None, grad_clip=None,
                 multi_precision=False, name=None):
        if learning_rate is None:
            raise ValueError("learning_rate should not be none")
        if batch_num is None or batch_num <= 0:
            raise ValueError("batch_num should be greater than 0")
        super().__init__(learning_rate, parameters, weight_decay, grad_clip, name, multi_precision)
        self._n = int(batch_num)
        self._state = {}

    def _apply(self, pgs, grad_scale):
        lr = self.get_lr()
        wd = self.regularization.coeff if isinstance(self.regularization, L2Decay) else 0.0
        for p, g, _ in pgs:
            w = p.as_subclass(torch.Tensor)
            g = g.as_subclass(torch.Tensor).to(w.dtype)
            if grad_scale is not None:
                g = g * grad_scale.to(g.dtype)
            st = self._state.get(p.name)
            if st is None:
                st = self._state[p.name] = {"d": torch.zeros_like(w), "y": torch.zeros((self._n, *w.shape), dtype=w.dtype,
                                                                                   device=w.device), "m": 0}
            i = st["m"] % self._n
            st["d"].add_(g - st["y"][i])
            st["y"][i].copy_(g)
            w.sub_(lr * (st["d"] / min(st["m"] + 1, self._n) + wd * w))
            st["m"] += 1


class LBFGS(Optimizer):
    """Limited-memory BFGS with optional strong-Wolfe line search; ``step(closure)`` re-evaluates the loss."""

    def __init__(self, learning_rate=1.0, max_iter=20, max_eval=None, tolerance_grad=1e-7, tolerance_change=1e-9,
                 history_size=100, line_search_fn=None, parameters=None, weight_decay=None, grad_clip=None, name=None):
        super().__init__(learning_rate, parameters, weight_decay, grad_clip, name)
        self._impl = torch.optim.LBFGS(self._parameter_list, lr=float(learning_rate), max_iter=max_iter, max_eval=max_eval,
                                       tolerance_grad=tolerance_grad, tolerance_change=tolerance_change,
                                       history_size=history_size, line_search_fn=line_search_fn)

    def step(self, closure):
        def wrapped():
            with torch.enable_grad():
                loss = closure()
            wd = self.regularization.coeff if isinstance(self.regularization, L2Decay) else 0.0
            if wd:
                for p in self._parameter_list:
                    if p.grad is not None:
                        p.grad.add_(p.detach(), alpha=wd)
            return loss.as_subclass(torch.Tensor) if isinstance(loss, torch.Tensor) else loss
        for grp in self._impl.param_groups:
            grp["lr"] = self.get_lr()
        from .._core.tensor import as_tensor
        return as_tensor(self._impl.step(wrapped))

    def state_dict(self):
        return {"_impl": self._impl.state_dict()}

    def set_state_dict(self, sd):
        if "_impl" in sd:
            self._impl.load_state_dict(sd["_impl"])
