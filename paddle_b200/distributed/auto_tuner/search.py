"""Search strategies of the auto tuner (python/paddle/distributed/auto_tuner/search.py:40-250): each walks a list of
candidate configurations and hands out the next one no pruning rule rejects."""
from __future__ import annotations

import logging
from abc import ABC, abstractmethod

from .prune import _PRUNE_FUNC, _PRUNE_HISTORY_FUNC
from .utils import gbs_search_all, load_configs_from_csv, search_all, search_by_dp_estimation

logger = logging.getLogger("auto_tuner")


class SearchAlgo(ABC):
    def __init__(self, tuner_cfg):
        self.tuner_cfg = tuner_cfg
        self.pruned_cfgs = []
        self.all_tasks = []
        self.idx = 0

    @abstractmethod
    def search_once(self, history_cfgs):
        ...

    def prune(self, tuner_cfg, cur_cfg, history_cfgs, pruned_cfgs=None):
        pruned_cfgs = self.pruned_cfgs if pruned_cfgs is None else pruned_cfgs
        for fn in _PRUNE_FUNC:
            if fn(tuner_cfg, cur_cfg, history_cfgs):
                return True
        for fn in _PRUNE_HISTORY_FUNC:
            if fn(tuner_cfg, cur_cfg, history_cfgs, pruned_cfgs):
                return True
        return False

    def _next(self, history_cfgs, tuner_cfg=None):
        tuner_cfg = tuner_cfg or self.tuner_cfg
        while self.idx < len(self.all_tasks):
            cfg = self.all_tasks[self.idx]
            self.idx += 1
            if self.prune(tuner_cfg, cfg, history_cfgs):
                self.pruned_cfgs.append(cfg)
                continue
            return cfg
        return None


class GridSearch(SearchAlgo):
    """Every combination of the candidates, fastest-expected first."""

    def __init__(self, tuner_cfg):
        super().__init__(tuner_cfg)
        self.all_tasks = search_all(tuner_cfg)
        algo = tuner_cfg.get("search_algo", {})
        if isinstance(algo, dict) and algo.get("sort") == "estimated":
            # try first what the analytic cost model expects to be fastest; what it expects not to fit is left out
            from .utils import sort_by_estimated_time
            self.all_tasks = sort_by_estimated_time(self.all_tasks, tuner_cfg)

    def search_once(self, history_cfgs):
        return self._next(history_cfgs)


class DpEstimationSearch(SearchAlgo):
    """Run the job without its data-parallel dimension on ``num_gpus / dp`` GPUs and scale the throughput by ``dp``:
    a 64-GPU search then needs 8-GPU trials only."""

    def __init__(self, tuner_cfg):
        super().__init__(tuner_cfg)
        self.all_tasks = search_by_dp_estimation(tuner_cfg)
        assert self.all_tasks, "data-parallel estimation found no configuration to run"

    def search_once(self, history_cfgs):
        while self.idx < len(self.all_tasks):
            cfg = self.all_tasks[self.idx]
            self.idx += 1
            small = dict(self.tuner_cfg)
            small["num_gpus"] = cfg["num_gpus"]
            small["candidates"] = None
            if self.prune(small, cfg, history_cfgs):
                self.pruned_cfgs.append(cfg)
                continue
            return cfg
        return None


class GBSSearch(SearchAlgo):
    """Grow the global batch on the fixed best shape until memory runs out."""

    def __init__(self, tuner_cfg):
        super().__init__(tuner_cfg)
        self.all_tasks = gbs_search_all(tuner_cfg)

    def search_once(self, history_cfgs):
        cfg = self._next(history_cfgs)
        if cfg is not None and history_cfgs and (history_cfgs[-1].get("max_mem_usage") == "OOM" or
                                                 history_cfgs[-1].get("error_info") == "OOM"):
            if cfg.get("global_batch_size", 0) > history_cfgs[-1].get("global_batch_size", 0):
                return None                              # the previous, smaller batch already did not fit
        return cfg


class CustomizeSearch(SearchAlgo):
    """Configurations listed by the user in a CSV (``tuner_cfg["search_algo"]["configs_csv"]``), in file order."""

    def __init__(self, tuner_cfg):
        super().__init__(tuner_cfg)
        path = tuner_cfg.get("configs_csv") or tuner_cfg.get("search_algo", {}).get("configs_csv")
        if not path:
            raise ValueError("customize search needs configs_csv")
        self.all_tasks = load_configs_from_csv(path)
        gbs = tuner_cfg.get("model_cfg", {}).get("global_batch_size")
        for c in self.all_tasks:
            if gbs is not None:
                c.setdefault("global_batch_size", gbs)

    def search_once(self, history_cfgs):
        return self._next(history_cfgs)


SEARCH_ALGOS = {"grid": GridSearch, "dp_estimation": DpEstimationSearch, "gbs": GBSSearch, "customize": CustomizeSearch}
