"""The tuner object the launcher drives (python/paddle/distributed/auto_tuner/tuner.py:23-200)."""
from __future__ import annotations

import os

from .recorder import HistoryRecorder
from .search import SEARCH_ALGOS
from .utils import default_candidates, gbs_default_candidates

_SHAPE_KEYS = ("dp_degree", "mp_degree", "pp_degree", "vpp_degree", "sharding_degree", "sharding_stage", "micro_batch_size",
               "use_recompute", "recompute_granularity", "global_batch_size")


class AutoTuner:
    """``search_once()`` hands out the next configuration that survives pruning; the caller runs it (for example
    through the launcher), reports the result with ``add_cfg`` and asks again until ``None``.

    ``tuner_cfg`` keys: ``num_gpus``, ``nodes``, ``model_cfg`` (hidden_size, num_layers, num_attention_heads,
    vocab_size, seq_length, global_batch_size), one entry per searched dimension (``"auto"``, a value or a list),
    ``search_algo`` (``{"name": "grid" | "dp_estimation" | "gbs" | "customize", ...}`` or the bare name),
    ``task_limit``, ``max_mem_usage`` (GB), ``metric_cfg`` (``name``, ``OptimizationDirection``), ``run_cmd``,
    ``invalid_strategy``."""

    def __init__(self, tuner_cfg):
        self.cur_task_id = 1
        self.task_limit = tuner_cfg.get("task_limit", 100)
        algo = tuner_cfg.get("search_algo", "grid")
        if isinstance(algo, str):
            algo = {"name": algo}
            tuner_cfg["search_algo"] = algo
        name = algo.get("name", "grid")
        if name not in SEARCH_ALGOS:
            raise NotImplementedError(f"search algorithm {name!r}; known: {sorted(SEARCH_ALGOS)}")
        if not tuner_cfg.get("candidates"):
            tuner_cfg["candidates"] = gbs_default_candidates(tuner_cfg) if name == "gbs" else default_candidates(tuner_cfg)
        self.tuner_cfg = tuner_cfg
        self.algo = SEARCH_ALGOS[name](tuner_cfg)
        self.history_cfgs = []
        self.resume_cfgs = []
        self.recorder = HistoryRecorder(tuner_cfg)

    # kept for callers of the first, flat version of this package
    @property
    def candidates(self):
        return self.algo.all_tasks

    def search_once(self):
        """Next configuration, or None when the space or the task limit is exhausted.  Configurations already present
        in a resumed history are skipped (their measured results were loaded with it)."""
        while self.cur_task_id <= self.task_limit:
            cfg = self.algo.search_once(self.history_cfgs)
            if cfg is None:
                return None
            done = self.get_cfg_from_resume(cfg)
            if done is not None:
                self.history_cfgs.append(done)
                continue
            self.cur_task_id += 1
            return cfg
        return None

    def add_cfg(self, cfg):
        """Record a finished (or failed) trial: pruning by history and the final ranking both read it."""
        self.history_cfgs.append(cfg)
        self.recorder.add_cfg(**cfg)

    def get_best(self):
        return self.recorder.get_best()[0]

    def store_history(self, path="./history.csv"):
        self.recorder.store_history(path)

    def resume_form_history(self, history_csv_path="./history.csv"):
        """Load the trials of an interrupted search; ``search_once`` will not hand them out again."""
        if not os.path.exists(history_csv_path):
            return False
        rows, err = HistoryRecorder(self.tuner_cfg).load_history(history_csv_path)
        if err:
            return False
        self.resume_cfgs = rows
        for r in rows:
            self.recorder.add_cfg(**r)
        return True

    resume_from_history = resume_form_history

    def get_cfg_from_resume(self, cur_cfg):
        """The recorded trial with the same shape as ``cur_cfg``, or None."""
        for r in self.resume_cfgs:
            if all(r.get(k) == cur_cfg.get(k) for k in _SHAPE_KEYS if k in cur_cfg and r.get(k) is not None):
                return r
        return None
