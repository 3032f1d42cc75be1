"""``HybridParallelOptimizer`` and ``HybridParallelClipGrad``
(python/paddle/distributed/fleet/meta_optimizers/dygraph_optimizer/hybrid_parallel_optimizer.py:48,275,524).

Global-norm clipping under hybrid parallelism: squared norms are summed separately for parameters that are
sharded over the mp group (``is_distributed``) and for replicated ones; the sharded part is all-reduced over
mp (and both over pp / sharding), then ``sqrt`` gives the global norm (:56-109,112-266).  The coefficient is
folded into the optimizer kernel, so gradients are read once.
"""
from __future__ import annotations

import torch

from .....nn.clip import ClipGradByGlobalNorm
from .... import collective as C
from ...utils.hybrid_parallel_util import (fused_allreduce_gradients, fused_allreduce_gradients_with_group,
                                           sharding_reduce_gradients)


class HybridParallelClipGrad:
    def __init__(self, clip, hcg):
        self._clip = clip
        self._hcg = hcg
        self.clip_norm = clip.clip_norm
        self._tables = {}

    def _sum_sq(self, key, grads):
        if not grads:
            return None
        if grads[0].is_cuda and all(g.is_contiguous() and g.dtype in (torch.float32, torch.bfloat16) for g in grads):
            from .....ops import native
            tab = self._tables.get(key)
            if tab is None or not tab.matches(grads, grads):
                tab = native.TensorTable(grads, grads)
                self._tables[key] = tab
            return tab.sq_l2_norm()
        return torch.stack([g.float().pow(2).sum() for g in grads]).sum().reshape(1)

    def global_norm_sq_pairs(self, params_grads):
        hcg = self._hcg
        dist, rep = [], []
        for p, g in params_grads:
            if g is None or not getattr(p, "need_clip", True):
                continue
            (dist if getattr(p, "is_distributed", False) else rep).append(g)
        dev = params_grads[0][1].device
        zero = torch.zeros(1, dtype=torch.float32, device=dev)
        d = self._sum_sq("dist", dist)
        r = self._sum_sq("rep", rep)
        d = zero.clone() if d is None else d
        r = zero.clone() if r is None else r
        mp = hcg.get_model_parallel_group()
        if mp is not None and mp.nranks > 1:
            C.all_reduce(d, group=mp)
        total = d + r
        pp = hcg.get_pipe_parallel_group()
        if pp is not None and pp.nranks > 1:
            C.all_reduce(total, group=pp)
        sh = hcg.get_sharding_parallel_group()
        if sh is not None and sh.nranks > 1 and getattr(self, "_sharded_grads", False):
            C.all_reduce(total, group=sh)
        return total

    def clip_coef(self, norm_sq):
        return self._clip.clip_coef(norm_sq)

    def __call__(self, params_grads):
        coef = self.clip_coef(self.global_norm_sq_pairs(params_grads))
        out = []
        for p, g in params_grads:
            if g is None or not getattr(p, "need_clip", True):
                out.append((p, g))
            else:
                out.append((p, g.mul_(coef.to(g.dtype))))
        return out

    _dygraph_clip = __call__

    def __getattr__(self, item):
        return getattr(self._clip, item)


class HybridParallelOptimizer:
    def __init__(self, optimizer, hcg, strategy):
        self._inner_opt = optimizer
        self._hcg = hcg
        self._strategy = strategy
        self._use_dp = hcg.get_data_parallel_world_size() > 1 or hcg.get_sep_parallel_world_size() > 1
        self._sharding_enable = hcg.get_sharding_parallel_world_size() > 1
        self._need_dp = self._use_dp
        mp_cfg = strategy.hybrid_configs["mp_configs"]
        self._sync_param = mp_cfg["sync_param"]
        self._sync_grad = mp_cfg["sync_grad"]
        self._sync_moment = mp_cfg["sync_moment"]
        if self._sharding_enable:
            from .dygraph_sharding_optimizer import DygraphShardingOptimizer, DygraphShardingOptimizerV2
            split = strategy.hybrid_configs["sharding_configs"]["split_param"]
            if split:
                self._inner_opt = DygraphShardingOptimizerV2(optimizer, hcg,
                                                             strategy.hybrid_configs["sharding_configs"])
            else:
                self._inner_opt = DygraphShardingOptimizer(optimizer, hcg)
        base = optimizer
        clip = base._grad_clip
        if isinstance(clip, ClipGradByGlobalNorm):
            hclip = HybridParallelClipGrad(clip, hcg)
            hclip._sharded_grads = self._sharding_enable
            base._grad_clip = clip  # keep type for isinstance checks in Optimizer.step
            base._global_norm_sq = lambda c, pgs, _h=hclip: _h.global_norm_sq_pairs(pgs)

    # ------------------------------------------------------------------
    def _hybrid_sync_grad(self, params):
        if self._sharding_enable:
            self._inner_opt.reduce_gradients(params, self._hcg)
        if self._need_dp:
            fused_allreduce_gradients(params, self._hcg)

    def _mp_sync(self, params):
        mp = self._hcg.get_model_parallel_group()
        if mp is None or mp.nranks == 1:
            return
        names = self._strategy.hybrid_configs["mp_configs"]["sync_param_name"]
        sel = [p for p in params if not getattr(p, "is_distributed", False) and any(n in p.name for n in names)]
        if self._sync_grad and sel:
            fused_allreduce_gradients_with_group(sel, mp, scale=1.0 / mp.nranks)
        return sel

    @torch.no_grad()
    def step(self):
        params = [p for p in self._inner_opt._parameter_list if p.requires_grad]
        self._hybrid_sync_grad(params)
        sel = self._mp_sync(params)
        self._inner_opt.step()
        if self._sync_param and sel:
            src = self._hcg.get_model_parallel_group_src_rank()
            for p in sel:
                C.broadcast(p.data, src, self._hcg.get_model_parallel_group())

    def minimize(self, loss, startup_program=None, parameters=None, no_grad_set=None):
        loss.backward()
        self.step()
        return None, None

    def clear_grad(self, set_to_zero=True):
        self._inner_opt.clear_grad(set_to_zero)

    clear_gradients = clear_grad

    def state_dict(self, *args, **kwargs):
        return self._inner_opt.state_dict(*args, **kwargs)

    def set_state_dict(self, sd):
        return self._inner_opt.set_state_dict(sd)

    def __getattr__(self, item):
        return getattr(self._inner_opt, item)
