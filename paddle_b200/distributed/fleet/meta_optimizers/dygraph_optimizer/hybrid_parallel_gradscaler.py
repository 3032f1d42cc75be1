"""GradScaler for hybrid-parallel training
(python/paddle/distributed/fleet/meta_optimizers/dygraph_optimizer/hybrid_parallel_gradscaler.py:29-96).

Every rank unscales and checks only the gradients it holds: a tensor-parallel rank its weight shards, a pipeline stage
its layers, a sharding rank its partition.  The step must be skipped everywhere when any of them saw an inf / nan, so
``found_inf`` is all-reduced (MAX) after the local check - over the whole job, as the reference does (:76-82; its comment
explains that the data-parallel gradient all-reduce runs after the scaler, hence the global group), or over the
``check`` group of the topology when only the model-parallel axes should agree (``use_check_group=True``).
The wrapper keeps the wrapped scaler's whole interface (``scale``, ``step``, ``update``, ``minimize``, ``unscale_``,
``state_dict`` ...)."""
from __future__ import annotations

import torch

from .... import collective as C


class HybridParallelGradScaler:
    def __init__(self, scaler, hcg, use_check_group=False):
        self._scaler = scaler
        self._hcg = hcg
        self._use_dp_mode = hcg is not None and hasattr(hcg, "get_parallel_mode") and _is_pure_dp(hcg)
        self._group = None
        if use_check_group and hcg is not None and hasattr(hcg, "get_check_parallel_group"):
            self._group = hcg.get_check_parallel_group()
        scaler._sync_found_inf = self._sync

    def _sync(self, found):
        """Agree on found_inf.  Pure data parallelism needs nothing: every rank holds all gradients, already averaged."""
        if self._use_dp_mode or not C.is_initialized() or C.get_world_size() == 1:
            return found
        t = found.to(torch.int32)
        C.all_reduce(t, C.ReduceOp.MAX, group=self._group)
        return t

    # the reference exposes these on the wrapper itself
    def scale(self, var):
        return self._scaler.scale(var)

    def unscale_(self, optimizer):
        return self._scaler.unscale_(optimizer)

    _unscale = unscale_

    def step(self, optimizer):
        return self._scaler.step(optimizer)

    def update(self):
        return self._scaler.update()

    def minimize(self, optimizer, *args, **kwargs):
        self._scaler.step(optimizer)
        self._scaler.update()
        return None, None

    def state_dict(self):
        return self._scaler.state_dict()

    def load_state_dict(self, sd):
        return self._scaler.load_state_dict(sd)

    def __getattr__(self, item):
        return getattr(self._scaler, item)


def _is_pure_dp(hcg):
    try:
        return (hcg.get_model_parallel_world_size() == 1 and hcg.get_pipe_parallel_world_size() == 1
                and hcg.get_sharding_parallel_world_size() == 1 and hcg.get_sep_parallel_world_size() == 1)
    except AttributeError:
        return False
