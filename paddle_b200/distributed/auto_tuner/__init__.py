"""``paddle.distributed.auto_tuner`` (python/paddle/distributed/auto_tuner/: tuner.py, search.py, prune.py,
recorder.py, cost_model.py, memory_cost_model.py, utils.py): enumerate hybrid-parallel configurations (dp / mp / pp /
vpp / sharding / micro-batch / recompute) for a given number of GPUs, prune the infeasible ones with divisibility
rules, a memory model and the results of earlier trials, build each trial's launcher command line, read its logs,
record measured results and report the best."""
from __future__ import annotations

from . import cost_model, memory_cost_model, prune, recorder, search, tuner, utils  # noqa: F401
from .cost_model import divisor, get_mem, get_not_oom_cfgs
from .prune import is_pruned, register_prune, register_prune_history
from .recorder import HistoryRecorder
from .search import CustomizeSearch, DpEstimationSearch, GBSSearch, GridSearch, SearchAlgo
from .tuner import AutoTuner
from .utils import (default_candidates, find_error_from_log, gen_new_args, load_configs_from_csv, read_log,
                    read_memory_log, read_metric_log, search_all)


def divisors(n):
    return divisor(n)


def memory_cost_gb(cfg, model):
    """GB per GPU of configuration ``cfg`` for ``model`` (num_layers, hidden_size, vocab_size, seq_length,
    num_attention_heads, global_batch_size) - the closed-form model of ``cost_model.get_mem``."""
    n = cfg["dp_degree"] * cfg["mp_degree"] * cfg["pp_degree"] * cfg.get("sharding_degree", 1)
    return get_mem(n, cfg, model["num_layers"], model["hidden_size"], model.get("num_attention_heads", model["hidden_size"] // 128),
                   model["vocab_size"], model.get("seq_length", 2048), cfg.get("global_batch_size", model.get("global_batch_size", 1)))


__all__ = ["AutoTuner", "HistoryRecorder", "SearchAlgo", "GridSearch", "DpEstimationSearch", "GBSSearch", "CustomizeSearch",
           "register_prune", "register_prune_history", "is_pruned", "default_candidates", "search_all", "gen_new_args",
           "read_log", "read_metric_log", "read_memory_log", "find_error_from_log", "load_configs_from_csv", "divisors",
           "divisor", "memory_cost_gb", "get_mem", "get_not_oom_cfgs"]
