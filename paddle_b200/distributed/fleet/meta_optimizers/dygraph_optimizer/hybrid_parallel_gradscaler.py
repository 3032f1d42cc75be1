"""GradScaler whose ``found_inf`` is agreed on by every rank
(python/paddle/distributed/fleet/meta_optimizers/dygraph_optimizer/hybrid_parallel_gradscaler.py:61-82)."""
from __future__ import annotations

from .... import collective as C


class HybridParallelGradScaler:
    def __init__(self, scaler, hcg):
        self._scaler = scaler
        self._hcg = hcg
        scaler._sync_found_inf = self._sync

    def _sync(self, found):
        C.all_reduce(found, C.ReduceOp.MAX, group=None)
        return found

    def __getattr__(self, item):
        return getattr(self._scaler, item)
