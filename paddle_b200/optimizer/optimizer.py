"""Optimizer base class with Paddle's state-dict layout.

State keys follow python/paddle/optimizer/optimizer.py: every accumulator is stored under its variable
name ``"{param.name}_{accumulator}_0"`` (``_add_accumulator:1030``), fp32 master weights under
``"master_weights"`` keyed by parameter name (``:413``), and the scheduler under ``"LR_Scheduler"``
(``:418``).  On GPU the update of a whole parameter group is one multi-tensor kernel launch.
"""
from __future__ import annotations

import collections

import numpy as np
import torch

from .._core.tensor import Tensor, as_tensor, to_tensor
from ..nn.clip import ClipGradByGlobalNorm
from .lr import LRScheduler


class L2Decay:
    def __init__(self, coeff=0.0):
        self.coeff = float(coeff)

    _regularization_coeff = property(lambda self: self.coeff)


class L1Decay(L2Decay):
    pass


class Optimizer:
    _accumulator_names: tuple = ()
    _handles_skip = False   # True when the update kernels read the device-side skip flag themselves

    def __init__(self, learning_rate=0.001, parameters=None, weight_decay=None, grad_clip=None, name=None,
                 multi_precision=False):
        if parameters is None:
            from ..static import graph as _sg
            if not _sg._S.enabled:
                raise ValueError("parameters must be given in dygraph mode")
            self._deferred_parameters = True      # static mode: minimize() collects the program's parameters
        parameters = list(parameters or [])
        self._param_groups = []
        if parameters and isinstance(parameters[0], dict):
            for g in parameters:
                g = dict(g)
                g["params"] = list(g["params"])
                self._param_groups.append(g)
        else:
            self._param_groups.append({"params": parameters})
        self._parameter_list = [p for g in self._param_groups for p in g["params"]]
        self._learning_rate = learning_rate
        self._weight_decay = weight_decay
        self.regularization = weight_decay if isinstance(weight_decay, L2Decay) else (
            L2Decay(weight_decay) if isinstance(weight_decay, (int, float)) else weight_decay)
        self._grad_clip = grad_clip
        self._multi_precision = multi_precision
        self._name = name
        self._accumulators = collections.defaultdict(dict)   # acc name -> {param.name: tensor}
        self._master_weights = {}
        self._accumulators_holder = {}
        self._step_count = 0
        self._tables = {}
        self._aux_grad_scale = None   # optional device scalar folded into the update (loss-scale inverse)
        self._skip_flag = None        # optional device int: nonzero -> skip the update (found_inf)

    # ------------------------------------------------------------------ lr
    def get_lr(self):
        lr = self._learning_rate
        return float(lr()) if isinstance(lr, LRScheduler) else float(lr)

    def set_lr(self, value):
        if isinstance(self._learning_rate, LRScheduler):
            raise RuntimeError("set_lr is not allowed when the learning rate is an LRScheduler")
        self._learning_rate = float(value)

    def set_lr_scheduler(self, scheduler):
        self._learning_rate = scheduler

    # ------------------------------------------------------------------ accumulators
    def _add_accumulator(self, name, param, dtype=None, fill_value=0.0, shape=None):
        if param.name in self._accumulators[name]:
            return self._accumulators[name][param.name]
        dtype = dtype or (torch.float32 if param.dtype in (torch.bfloat16, torch.float16) else param.dtype)
        # a distributed parameter reports its global shape; state lives on the local shard
        shape = list(getattr(param, "_local_shape", param.shape)) if shape is None else shape
        t = as_tensor(torch.full(shape, fill_value, dtype=dtype, device=param.device))
        t.name = f"{param.name}_{name}_0"
        held = self._accumulators_holder.pop(t.name, None)
        if held is not None:
            t.copy_(held.to(t.device).to(t.dtype).reshape(t.shape))
        self._accumulators[name][param.name] = t
        return t

    def _get_accumulator(self, name, param):
        return self._accumulators[name][param.name]

    def _use_master(self, p):
        return self._multi_precision and p.dtype in (torch.bfloat16, torch.float16)

    def _create_master_weight(self, param):
        mw = self._master_weights.get(param.name)
        if mw is None:
            mw = as_tensor(param.detach().to(torch.float32).clone())
            mw.name = f"{param.name}_fp32_master_0"
            held = self._accumulators_holder.get("master_weights", {}).pop(param.name, None) \
                if isinstance(self._accumulators_holder.get("master_weights"), dict) else None
            if held is not None:
                mw.copy_(held.to(mw.device).to(torch.float32).reshape(mw.shape))
            self._master_weights[param.name] = mw
        return mw

    def _create_accumulators(self, params):
        pass

    # ------------------------------------------------------------------ step
    @staticmethod
    def _grad_of(p):
        mg = getattr(p, "main_grad", None)
        return mg if mg is not None else p.grad

    def _collect(self):
        out = []
        for group in self._param_groups:
            for p in group["params"]:
                if not p.requires_grad:
                    continue
                g = self._grad_of(p)
                if g is not None:
                    out.append((p, g, group))
        return out

    @torch.no_grad()
    def step(self):
        pgs = self._collect()
        if not pgs:
            return
        if self._skip_flag is not None and not self._handles_skip and int(self._skip_flag.item()) != 0:
            return
        self._create_accumulators([p for p, _, _ in pgs])
        grad_scale = self._aux_grad_scale
        clip = self._grad_clip
        if clip is not None:
            if isinstance(clip, ClipGradByGlobalNorm):
                # fold the clip coefficient into the update kernel: no extra pass over the gradients
                sel = [g for p, g, _ in pgs if getattr(p, "need_clip", True)]
                coef = clip.clip_coef(self._global_norm_sq(clip, [(p, g) for p, g, _ in pgs])) if sel else None
                if coef is not None:
                    grad_scale = coef if grad_scale is None else coef * grad_scale
            else:
                clipped = clip([(p, g) for p, g, _ in pgs])
                pgs = [(p, g, grp) for (p, g), (_, _, grp) in zip(clipped, pgs)]
        self._step_count += 1
        self._apply(pgs, grad_scale)

    def _global_norm_sq(self, clip, params_grads):
        return clip.global_norm_sq([g for p, g in params_grads if getattr(p, "need_clip", True)])

    def _apply(self, pgs, grad_scale):
        raise NotImplementedError

    def _set_parameters(self, parameters):
        self._param_groups = [{"params": list(parameters)}]
        self._parameter_list = list(parameters)

    def minimize(self, loss, startup_program=None, parameters=None, no_grad_set=None):
        from ..static import graph as _sg
        if _sg.recording():
            from ..static import _static_minimize
            return _static_minimize(self, loss, parameters, no_grad_set)
        # dynamic mode: the caller has already run ``loss.backward()``; minimize applies the gradients that exist
        # (python/paddle/optimizer/optimizer.py ``minimize`` -> ``backward`` collects ``param.grad`` in dygraph)
        params_grads = self.backward(loss, parameters=parameters, no_grad_set=no_grad_set)
        if not params_grads and loss is not None and getattr(loss, "grad_fn", None) is not None:
            loss.backward()
        self.step()
        return None, params_grads

    def backward(self, loss=None, startup_program=None, parameters=None, no_grad_set=None, callbacks=None):
        """(parameter, gradient) pairs of the parameters that have a gradient (dynamic mode: the gradients computed by the
        caller's ``loss.backward()``)."""
        skip = set(id(p) for p in (no_grad_set or []))
        plist = parameters if parameters is not None else self._parameter_list
        flat = []
        for p in plist:
            flat += list(p["params"]) if isinstance(p, dict) else [p]
        return [(p, p.grad) for p in flat if p.grad is not None and id(p) not in skip and not p.stop_gradient]

    def apply_gradients(self, params_grads):
        """Update the given parameters with the given gradients."""
        for p, g in params_grads:
            if g is not None and p.grad is not g:
                p.grad = g if isinstance(g, torch.Tensor) else torch.as_tensor(g)
        self.step()
        return []

    def clear_grad(self, set_to_zero=True):
        for p in self._parameter_list:
            if set_to_zero:
                if p.grad is not None:
                    p.grad.zero_()
                mg = getattr(p, "main_grad", None)
                if mg is not None:
                    mg.zero_()
            else:
                p.grad = None
                if getattr(p, "main_grad", None) is not None and not getattr(p, "_main_grad_persistent", False):
                    p.main_grad = None
                elif getattr(p, "main_grad", None) is not None:
                    p.main_grad.zero_()

    clear_gradients = clear_grad

    # ------------------------------------------------------------------ state dict
    def state_dict(self):
        sd = {}
        for acc, d in self._accumulators.items():
            for pname, t in d.items():
                sd[t.name] = t
        if self._master_weights:
            sd["master_weights"] = dict(self._master_weights)
        if isinstance(self._learning_rate, LRScheduler):
            sd["LR_Scheduler"] = self._learning_rate.state_dict()
        return sd

    def set_state_dict(self, state_dict):
        state_dict = dict(state_dict)
        if isinstance(self._learning_rate, LRScheduler) and "LR_Scheduler" in state_dict:
            self._learning_rate.set_state_dict(state_dict.pop("LR_Scheduler"))
        state_dict.pop("LR_Scheduler", None)

        def _t(v):
            return v if isinstance(v, torch.Tensor) else to_tensor(np.asarray(v))
        mw = state_dict.pop("master_weights", None)
        if mw is not None:
            for k, v in mw.items():
                v = _t(v)
                if k in self._master_weights:
                    self._master_weights[k].copy_(v.to(self._master_weights[k].device).float())
                else:
                    self._accumulators_holder.setdefault("master_weights", {})[k] = v
        existing = {t.name: t for d in self._accumulators.values() for t in d.values()}
        for k, v in state_dict.items():
            if str(k).endswith("@@"):
                continue
            v = _t(v)
            if k in existing:
                existing[k].copy_(v.to(existing[k].device).to(existing[k].dtype).reshape(existing[k].shape))
            else:
                self._accumulators_holder[k] = v
        # step count is recoverable from beta1_pow_acc when present (AdamW family)
        self._restore_step_from_state()

    set_dict = set_state_dict
    load_state_dict = set_state_dict

    def _restore_step_from_state(self):
        pass

    def _table(self, key, params, grads, masters=None, ms=None, vs=None):
        from ..ops import native
        tab = self._tables.get(key)
        if tab is None or not tab.matches(params, grads):
            tab = native.TensorTable(params, grads, masters, ms, vs)
            self._tables[key] = tab
        return tab
