"""Adam / AdamW (python/paddle/optimizer/adam.py, adamw.py:168-172,528).

Update rule (paddle/phi/kernels/gpu/adamw_kernel.cu:62-93), all in fp32:
    p *= 1 - lr * coeff ;  m = b1 m + (1-b1) g ;  v = b2 v + (1-b2) g^2
    p -= lr / (1 - b1^t) * m / (sqrt(v) / sqrt(1 - b2^t) + eps)
"""
from __future__ import annotations

import math

import torch

from .optimizer import L2Decay, Optimizer


class AdamW(Optimizer):
    _accumulator_names = ("moment1", "moment2", "beta1_pow_acc", "beta2_pow_acc")
    _handles_skip = True

    def __init__(self, learning_rate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8, parameters=None, weight_decay=0.01,
                 lr_ratio=None, apply_decay_param_fun=None, grad_clip=None, lazy_mode=False, multi_precision=False,
                 amsgrad=False, name=None):
        super().__init__(learning_rate, parameters, None, grad_clip, name, multi_precision)
        self._beta1, self._beta2, self._epsilon = float(beta1), float(beta2), float(epsilon)
        self._coeff = float(weight_decay.coeff if isinstance(weight_decay, L2Decay) else (weight_decay or 0.0))
        self._lr_ratio = lr_ratio
        self._apply_decay_param_fun = apply_decay_param_fun
        self._decoupled = True

    def _create_accumulators(self, params):
        for p in params:
            if self._use_master(p):
                self._create_master_weight(p)
            self._add_accumulator("moment1", p)
            self._add_accumulator("moment2", p)
            self._add_accumulator("beta1_pow_acc", p, dtype=torch.float32, fill_value=self._beta1, shape=[1])
            self._add_accumulator("beta2_pow_acc", p, dtype=torch.float32, fill_value=self._beta2, shape=[1])

    def _restore_step_from_state(self):
        for name, t in list(self._accumulators_holder.items()):
            if isinstance(name, str) and name.endswith("_beta1_pow_acc_0") and self._beta1 not in (0.0, 1.0):
                v = float(t.reshape(-1)[0])
                if 0 < v < 1:
                    self._step_count = max(self._step_count, int(round(math.log(v) / math.log(self._beta1))) - 1)

    def _decay_for(self, p, group):
        coeff = group.get("weight_decay", self._coeff)
        coeff = float(coeff.coeff if isinstance(coeff, L2Decay) else coeff)
        if self._apply_decay_param_fun is not None and not self._apply_decay_param_fun(p.name):
            coeff = 0.0
        return coeff

    def _apply(self, pgs, grad_scale):
        base_lr = self.get_lr()
        t = self._step_count
        b1p, b2p = self._beta1 ** t, self._beta2 ** t
        buckets = {}
        for p, g, group in pgs:
            lr = base_lr * group.get("learning_rate", 1.0) * p.optimize_attr.get("learning_rate", 1.0)
            if self._lr_ratio is not None:
                lr *= self._lr_ratio(p)
            coeff = self._decay_for(p, group)
            buckets.setdefault((lr, coeff, p.device.type), []).append((p, g))
        for bi, ((lr, coeff, devt), items) in enumerate(sorted(buckets.items(), key=lambda kv: (kv[0][1], kv[0][0]))):
            params = [p for p, _ in items]
            grads = [g for _, g in items]
            ms = [self._accumulators["moment1"][p.name] for p in params]
            vs = [self._accumulators["moment2"][p.name] for p in params]
            masters = [self._master_weights.get(p.name) for p in params]
            native_ok = devt == "cuda" and all(
                p.dtype in (torch.float32, torch.bfloat16) and g.dtype in (torch.float32, torch.bfloat16)
                and p.is_contiguous() and g.is_contiguous() and (p.dtype == torch.float32 or m_ is not None)
                for p, g, m_ in zip(params, grads, masters))
            if native_ok:
                tab = self._table(("adamw", coeff, len(params), bi), params, grads, masters, ms, vs)
                tab.adamw(lr, self._beta1, self._beta2, self._epsilon, coeff if self._decoupled else 0.0, b1p, b2p,
                          grad_scale, self._skip_flag)
            else:
                self._apply_torch(params, grads, masters, ms, vs, lr, coeff, b1p, b2p, grad_scale)
        for p, _, _ in pgs:  # keep the checkpoint-visible beta powers in step with the host counter
            self._accumulators["beta1_pow_acc"][p.name].fill_(b1p * self._beta1)
            self._accumulators["beta2_pow_acc"][p.name].fill_(b2p * self._beta2)

    def _apply_torch(self, params, grads, masters, ms, vs, lr, coeff, b1p, b2p, grad_scale):
        if self._skip_flag is not None and int(self._skip_flag.item()) != 0:
            return
        for p, g, mw, m, v in zip(params, grads, masters, ms, vs):
            gf = g.float()
            if grad_scale is not None:
                gf = gf * grad_scale.to(gf.device)
            w = mw if mw is not None else p.data.float()
            if self._decoupled:
                w.mul_(1.0 - lr * coeff)
            elif coeff:
                gf = gf + coeff * w
            m.mul_(self._beta1).add_(gf, alpha=1 - self._beta1)
            v.mul_(self._beta2).addcmul_(gf, gf, value=1 - self._beta2)
            denom = v.sqrt() / math.sqrt(1 - b2p) + self._epsilon
            w.addcdiv_(m, denom, value=-(lr / (1 - b1p)))
            if mw is not None or p.dtype != torch.float32:
                p.data.copy_(w)


class Adam(AdamW):
    """Adam with (optional) L2 regularisation folded into the gradient instead of decoupled decay."""

    def __init__(self, learning_rate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8, parameters=None, weight_decay=None,
                 grad_clip=None, lazy_mode=False, multi_precision=False, use_multi_tensor=False, amsgrad=False,
                 name=None):
        super().__init__(learning_rate, beta1, beta2, epsilon, parameters, weight_decay or 0.0, None, None, grad_clip,
                         lazy_mode, multi_precision, amsgrad, name)
        self._decoupled = False

    def _apply(self, pgs, grad_scale):
        if self._coeff:
            pgs = [(p, (g.float() + self._coeff * (self._master_weights.get(p.name, p)).float()).to(g.dtype), grp)
                   for p, g, grp in pgs]
        saved, self._coeff = self._coeff, 0.0
        try:
            super()._apply(pgs, grad_scale)
        finally:
            self._coeff = saved


class Adamax(Optimizer):
    def __init__(self, learning_rate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8, parameters=None, weight_decay=None,
                 grad_clip=None, name=None, multi_precision=False):
        super().__init__(learning_rate, parameters, weight_decay, grad_clip, name, multi_precision)
        self._beta1, self._beta2, self._epsilon = float(beta1), float(beta2), float(epsilon)

    def _create_accumulators(self, params):
        for p in params:
            self._add_accumulator("moment", p)
            self._add_accumulator("inf_norm", p)

    def _apply(self, pgs, grad_scale):
        lr, t = self.get_lr(), self._step_count
        for p, g, _ in pgs:
            gf = g.float() * (grad_scale if grad_scale is not None else 1.0)
            m, u = self._accumulators["moment"][p.name], self._accumulators["inf_norm"][p.name]
            m.mul_(self._beta1).add_(gf, alpha=1 - self._beta1)
            torch.maximum(u * self._beta2, gf.abs() + self._epsilon, out=u)
            p.data.add_((-(lr / (1 - self._beta1 ** t)) * m / u).to(p.dtype))
