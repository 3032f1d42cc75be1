"""SGD / Momentum / RMSProp / Adagrad / Adadelta / Lamb (python/paddle/optimizer/*.py)."""
from __future__ import annotations

import torch

from .optimizer import L2Decay, Optimizer


class Momentum(Optimizer):
    def __init__(self, learning_rate=0.001, momentum=0.9, parameters=None, use_nesterov=False, weight_decay=None,
                 grad_clip=None, multi_precision=False, rescale_grad=1.0, use_multi_tensor=False, name=None):
        super().__init__(learning_rate, parameters, weight_decay, grad_clip, name, multi_precision)
        self._momentum, self._nesterov = float(momentum), bool(use_nesterov)
        self._use_momentum = True

    def _create_accumulators(self, params):
        for p in params:
            if self._use_master(p):
                self._create_master_weight(p)
            if self._use_momentum:
                self._add_accumulator("velocity", p)

    def _apply(self, pgs, grad_scale):
        lr = self.get_lr()
        wd = self.regularization.coeff if isinstance(self.regularization, L2Decay) else 0.0
        params = [p for p, _, _ in pgs]
        grads = [g for _, g, _ in pgs]
        masters = [self._master_weights.get(p.name) for p in params]
        vel = [self._accumulators["velocity"][p.name] for p in params] if self._use_momentum else None
        native_ok = params[0].is_cuda and all(
            p.dtype in (torch.float32, torch.bfloat16) and g.dtype in (torch.float32, torch.bfloat16)
            and p.is_contiguous() and g.is_contiguous() and (p.dtype == torch.float32 or m is not None)
            for p, g, m in zip(params, grads, masters))
        if native_ok:
            tab = self._table(("mom", len(params)), params, grads, masters, vel, None)
            tab.momentum(lr, self._momentum, wd, self._nesterov, self._use_momentum, grad_scale)
            return
        for i, (p, g) in enumerate(zip(params, grads)):
            w = masters[i] if masters[i] is not None else p.data
            gf = g.to(w.dtype)
            if grad_scale is not None:
                gf = gf * grad_scale.to(gf.device).to(gf.dtype)
            if wd:
                gf = gf + wd * w
            if self._use_momentum:
                v = vel[i]
                v.mul_(self._momentum).add_(gf)
                w.add_(gf + self._momentum * v if self._nesterov else v, alpha=-lr)
            else:
                w.add_(gf, alpha=-lr)
            if masters[i] is not None:
                p.data.copy_(w)


class SGD(Momentum):
    def __init__(self, learning_rate=0.001, parameters=None, weight_decay=None, grad_clip=None, multi_precision=False,
                 name=None):
        super().__init__(learning_rate, 0.0, parameters, False, weight_decay, grad_clip, multi_precision)
        self._use_momentum = False


class _TorchBacked(Optimizer):
    """Less common optimizers delegate the arithmetic to the torch implementation of the same rule."""
    _cls = None

    def __init__(self, learning_rate=0.001, parameters=None, weight_decay=None, grad_clip=None, name=None, **kw):
        super().__init__(learning_rate, parameters, weight_decay, grad_clip, name)
        self._kw = kw
        self._impl = None

    def _apply(self, pgs, grad_scale):
        if self._impl is None:
            wd = self.regularization.coeff if isinstance(self.regularization, L2Decay) else 0.0
            self._impl = self._cls(self._parameter_list, lr=self.get_lr(), weight_decay=wd, **self._kw)
        for grp in self._impl.param_groups:
            grp["lr"] = self.get_lr()
        if grad_scale is not None:
            for p, g, _ in pgs:
                g.mul_(grad_scale.to(g.dtype))
        self._impl.step()

    def state_dict(self):
        sd = super().state_dict()
        if self._impl is not None:
            sd["_impl"] = self._impl.state_dict()
        return sd


class RMSProp(_TorchBacked):
    _cls = torch.optim.RMSprop

    def __init__(self, learning_rate, rho=0.95, epsilon=1e-6, momentum=0.0, centered=False, parameters=None,
                 weight_decay=None, grad_clip=None, name=None):
        super().__init__(learning_rate, parameters, weight_decay, grad_clip, name, alpha=rho, eps=epsilon,
                         momentum=momentum, centered=centered)


class Adagrad(_TorchBacked):
    _cls = torch.optim.Adagrad

    def __init__(self, learning_rate, epsilon=1e-6, parameters=None, weight_decay=None, grad_clip=None, name=None,
                 initial_accumulator_value=0.0):
        super().__init__(learning_rate, parameters, weight_decay, grad_clip, name, eps=epsilon,
                         initial_accumulator_value=initial_accumulator_value)


class Adadelta(_TorchBacked):
    _cls = torch.optim.Adadelta

    def __init__(self, learning_rate=0.001, epsilon=1e-6, rho=0.95, parameters=None, weight_decay=None,
                 grad_clip=None, name=None):
        super().__init__(learning_rate, parameters, weight_decay, grad_clip, name, eps=epsilon, rho=rho)


class Lamb(Optimizer):
    """Layer-wise adaptive moments (python/paddle/optimizer/lamb.py)."""

    def __init__(self, learning_rate=0.001, lamb_weight_decay=0.01, beta1=0.9, beta2=0.999, epsilon=1e-6,
                 parameters=None, grad_clip=None, exclude_from_weight_decay_fn=None, multi_precision=False, name=None):
        super().__init__(learning_rate, parameters, None, grad_clip, name, multi_precision)
        self._wd, self._beta1, self._beta2, self._epsilon = float(lamb_weight_decay), float(beta1), float(beta2), float(epsilon)
        self._exclude = exclude_from_weight_decay_fn

    def _create_accumulators(self, params):
        for p in params:
            if self._use_master(p):
                self._create_master_weight(p)
            self._add_accumulator("moment1", p)
            self._add_accumulator("moment2", p)

    def _apply(self, pgs, grad_scale):
        lr, t = self.get_lr(), self._step_count
        for p, g, _ in pgs:
            w = self._master_weights.get(p.name)
            w = w if w is not None else p.data
            gf = g.float() * (grad_scale if grad_scale is not None else 1.0)
            m, v = self._accumulators["moment1"][p.name], self._accumulators["moment2"][p.name]
            m.mul_(self._beta1).add_(gf, alpha=1 - self._beta1)
            v.mul_(self._beta2).addcmul_(gf, gf, value=1 - self._beta2)
            mh, vh = m / (1 - self._beta1 ** t), v / (1 - self._beta2 ** t)
            wd = 0.0 if (self._exclude is not None and self._exclude(p)) else self._wd
            r = mh / (vh.sqrt() + self._epsilon) + wd * w.float()
            wn, rn = w.float().norm(), r.norm()
            trust = torch.where((wn > 0) & (rn > 0), wn / rn, torch.ones_like(wn))
            w.add_((-lr * trust * r).to(w.dtype))
            if w is not p.data:
                p.data.copy_(w)
