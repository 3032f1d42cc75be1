"""``paddle.distributed.auto_tuner`` (python/paddle/distributed/auto_tuner/: tuner.py, search.py, prune.py,
recorder.py, memory_cost_model.py): enumerate hybrid-parallel configurations (dp / mp / pp / sharding / micro-batch
/ recompute) for a given number of GPUs, prune the infeasible ones with divisibility rules and a memory model,
record measured results and report the best."""
from __future__ import annotations

import csv
import itertools


def divisors(n):
    return [d for d in range(1, n + 1) if n % d == 0]


def memory_cost_gb(cfg, model):
    """Rough bytes per GPU: bf16 weights + fp32 master/moments (sharded by sharding stage) + fp32 gradients +
    activations of the in-flight micro-batches (memory_cost_model.py)."""
    L, H, V, S = model["num_layers"], model["hidden_size"], model["vocab_size"], model["seq_length"]
    F = model.get("intermediate_size", 4 * H)
    params = L * (4 * H * H + 3 * H * F) + V * H
    p_local = params / (cfg["mp_degree"] * cfg["pp_degree"])
    shard = cfg["sharding_degree"]
    stage = cfg.get("sharding_stage", 1)
    weights = 2 * p_local / (shard if stage >= 3 else 1)
    grads = 4 * p_local / (shard if stage >= 2 else 1)
    opt = 12 * p_local / (shard if stage >= 1 else 1)
    per_layer_act = S * cfg["micro_batch_size"] * H * (34 if not cfg.get("use_recompute") else 2) / cfg["mp_degree"]
    in_flight = cfg["pp_degree"]
    acts = per_layer_act * (L / cfg["pp_degree"]) * in_flight
    return (weights + grads + opt + acts) / 2 ** 30


def default_candidates(tuner_cfg):
    n = tuner_cfg["num_gpus"]
    model = tuner_cfg["model_cfg"]
    gbs = model["global_batch_size"]
    cands = []
    for mp, pp in itertools.product(divisors(min(n, 8)), divisors(n)):
        if n % (mp * pp):
            continue
        rest = n // (mp * pp)
        for sharding in divisors(rest):
            dp = rest // sharding
            for mbs in tuner_cfg.get("micro_batch_size", [1, 2, 4, 8]):
                for stage in tuner_cfg.get("sharding_stage", [1]):
                    for rc in tuner_cfg.get("use_recompute", [False, True]):
                        cands.append(dict(dp_degree=dp, mp_degree=mp, pp_degree=pp, sharding_degree=sharding,
                                          sharding_stage=stage, micro_batch_size=mbs, use_recompute=rc,
                                          global_batch_size=gbs))
    return cands


_PRUNES = []


def register_prune(fn):
    _PRUNES.append(fn)
    return fn


@register_prune
def prune_by_divisibility(tuner_cfg, cfg, history):
    m = tuner_cfg["model_cfg"]
    if m["num_attention_heads"] % cfg["mp_degree"] or m["vocab_size"] % cfg["mp_degree"]:
        return True
    if m["num_layers"] % cfg["pp_degree"]:
        return True
    per_dp = cfg["global_batch_size"] / (cfg["dp_degree"] * cfg["sharding_degree"])
    return per_dp < cfg["micro_batch_size"] or per_dp % cfg["micro_batch_size"] != 0


@register_prune
def prune_by_memory(tuner_cfg, cfg, history):
    limit = tuner_cfg.get("max_mem_usage_gb", 180.0)
    return memory_cost_gb(cfg, tuner_cfg["model_cfg"]) > limit


@register_prune
def prune_by_history(tuner_cfg, cfg, history):
    """A configuration that needs at least the memory of one that already ran out of memory is skipped."""
    for h in history:
        if h.get("error") == "OOM" and all(cfg[k] == h[k] for k in ("mp_degree", "pp_degree", "sharding_degree", "sharding_stage")) \
                and cfg["micro_batch_size"] >= h["micro_batch_size"] and cfg["use_recompute"] <= h["use_recompute"]:
            return True
    return False


class HistoryRecorder:
    def __init__(self, metric="tokens_per_second", direction="max"):
        self.history, self.metric, self.direction = [], metric, direction

    def add_cfg(self, **cfg):
        self.history.append(dict(cfg))

    def sort_metric(self):
        ok = [h for h in self.history if h.get(self.metric) is not None]
        return sorted(ok, key=lambda h: h[self.metric], reverse=self.direction == "max")

    def get_best(self):
        s = self.sort_metric()
        return (s[0], False) if s else (None, True)

    def store_history(self, path="./history.csv"):
        keys = sorted({k for h in self.history for k in h})
        with open(path, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=keys)
            w.writeheader()
            w.writerows(self.history)

    def load_history(self, path="./history.csv"):
        with open(path) as f:
            self.history = [dict(r) for r in csv.DictReader(f)]
        return self.history, False


class AutoTuner:
    """``search_once()`` hands out the next configuration that survives pruning; the caller runs it (for example
    through the launcher), reports the result with ``add_cfg`` and asks again until ``None``."""

    def __init__(self, tuner_cfg):
        self.tuner_cfg = tuner_cfg
        self.candidates = default_candidates(tuner_cfg)
        self.recorder = HistoryRecorder(tuner_cfg.get("metric_cfg", {}).get("name", "tokens_per_second"),
                                        tuner_cfg.get("metric_cfg", {}).get("OptimizationDirection", "max").lower()[:3])
        self.idx = 0
        self.task_limit = tuner_cfg.get("task_limit", 100)
        self.handed_out = 0

    def search_once(self):
        while self.idx < len(self.candidates) and self.handed_out < self.task_limit:
            cfg = self.candidates[self.idx]
            self.idx += 1
            if any(p(self.tuner_cfg, cfg, self.recorder.history) for p in _PRUNES):
                continue
            self.handed_out += 1
            return cfg
        return None

    def add_cfg(self, cfg):
        self.recorder.add_cfg(**cfg)

    def get_best(self):
        return self.recorder.get_best()[0]
