"""Search-space helpers, launcher-argument generation and log reading of the auto tuner
(python/paddle/distributed/auto_tuner/utils.py:36-1700)."""
from __future__ import annotations

import copy
import csv
import itertools
import os
import re

from .cost_model import divisor

__SUPPORTED_RECOMPUTE_GRANULARITY__ = ["full", "full_attn", "core_attn"]
_DEGREE_KEYS = ("dp_degree", "mp_degree", "pp_degree", "sharding_degree")
_SPACE_KEYS = ("dp_degree", "sharding_degree", "sharding_stage", "mp_degree", "pp_degree", "vpp_degree",
               "micro_batch_size", "use_recompute", "recompute_granularity")


def dist_degree(mode, num_gpus, num_nodes, tuner_cfg=None):
    """Candidate degrees of one parallel dimension: every divisor of the GPU count, with the usual placement rules -
    tensor parallelism stays inside a node (NVLink domain), pipeline stages are at least one per node when ``pp`` spans
    nodes."""
    assert mode in ("dp", "mp", "pp", "sharding", "mbs", "vpp")
    per_node = max(1, num_gpus // max(1, num_nodes))
    if mode == "mp":
        return [d for d in divisor(num_gpus, reverse=True) if d <= per_node]
    if mode == "pp":
        out = divisor(num_gpus)
        if num_nodes > 1 and tuner_cfg and tuner_cfg.get("pp_cross_node_only"):
            out = [d for d in out if d % num_nodes == 0 or d == 1]
        return out
    if mode in ("dp", "sharding"):
        return divisor(num_gpus, reverse=mode == "sharding")
    raise ValueError(f"{mode} has no degree candidates derived from the GPU count")


def _as_list(v):
    return list(v) if isinstance(v, (list, tuple)) else [v]


def default_candidates(tuner_cfg):
    """Fill every searchable key of ``tuner_cfg`` with a candidate list: ``"auto"`` expands to the defaults, a scalar
    becomes a one-element list, a list is kept, an absent key gets its neutral value."""
    cand = {}
    n = tuner_cfg["num_gpus"]
    nodes = tuner_cfg.get("nodes", tuner_cfg.get("num_nodes", 1))
    model = tuner_cfg.get("model_cfg", {})
    for mode, key in (("dp", "dp_degree"), ("mp", "mp_degree"), ("pp", "pp_degree"), ("sharding", "sharding_degree")):
        v = tuner_cfg.get(key)
        if v == "auto":
            cand[key] = dist_degree(mode, n, nodes, tuner_cfg)
        elif v is None:
            cand[key] = [1]
        else:
            cand[key] = _as_list(v)
    v = tuner_cfg.get("sharding_stage")
    cand["sharding_stage"] = [3, 2, 1] if v == "auto" else ([1] if v is None else _as_list(v))
    v = tuner_cfg.get("use_recompute")
    cand["use_recompute"] = [False, True] if v == "auto" else ([False] if v is None else _as_list(v))
    v = tuner_cfg.get("recompute_granularity")
    cand["recompute_granularity"] = list(__SUPPORTED_RECOMPUTE_GRANULARITY__) if v == "auto" else ([None] if v is None else _as_list(v))
    v = tuner_cfg.get("vpp_degree")
    layers = model.get("num_layers")
    cand["vpp_degree"] = (divisor(layers) if layers else [1]) if v == "auto" else ([1] if v is None else _as_list(v))
    v = tuner_cfg.get("micro_batch_size")
    gbs = model.get("global_batch_size")
    if v == "auto":
        cand["micro_batch_size"] = divisor(gbs) if gbs else [1, 2, 4, 8]
    elif v is None:
        cand["micro_batch_size"] = [1, 2, 4, 8] if "micro_batch_size" not in tuner_cfg else [1]
    else:
        cand["micro_batch_size"] = _as_list(v)
    for key, vals in (tuner_cfg.get("custom_search_dim") or {}).items():
        cand[key] = _as_list(vals.get("value", vals) if isinstance(vals, dict) else vals)
    return cand


def search_all(tuner_cfg):
    """Every combination of the candidates whose degrees multiply to the number of GPUs, as dicts, ordered so that the
    configurations expected to be fastest on an NVLink node come first: less pipeline, then less tensor parallelism,
    larger micro-batches, no recompute."""
    cand = tuner_cfg.get("candidates") or default_candidates(tuner_cfg)
    n = tuner_cfg["num_gpus"]
    keys = [k for k in _SPACE_KEYS if k in cand] + [k for k in cand if k not in _SPACE_KEYS]
    gbs = tuner_cfg.get("model_cfg", {}).get("global_batch_size")
    out = []
    for combo in itertools.product(*(cand[k] for k in keys)):
        cfg = dict(zip(keys, combo))
        prod = 1
        for k in _DEGREE_KEYS:
            prod *= cfg[k]
        if prod != n:
            continue
        if gbs is not None:
            cfg["global_batch_size"] = gbs
        if not cfg.get("use_recompute") and cfg.get("recompute_granularity") not in (None, cand["recompute_granularity"][0]):
            continue                                    # granularity is meaningless without recompute: keep one copy
        out.append(cfg)
    out.sort(key=lambda c: (c["pp_degree"], c["mp_degree"], -c["micro_batch_size"], bool(c.get("use_recompute")),
                            c.get("sharding_stage", 1)))
    return out


def search_by_dp_estimation(tuner_cfg):
    """Configurations for the data-parallel estimation mode: the job is run with ``dp = 1`` on ``num_gpus / dp`` GPUs
    and its throughput multiplied up, so only the (mp, pp, sharding) shapes of the smaller job are enumerated."""
    results = []
    for cfg in search_all(tuner_cfg):
        small = dict(cfg)
        small["estimated_dp_degree"] = cfg["dp_degree"]
        small["dp_degree"] = 1
        small["num_gpus"] = tuner_cfg["num_gpus"] // cfg["dp_degree"]
        if gbs := cfg.get("global_batch_size"):
            if gbs % cfg["dp_degree"]:
                continue
            small["global_batch_size"] = gbs // cfg["dp_degree"]
        key = tuple(sorted((k, str(v)) for k, v in small.items() if k != "estimated_dp_degree"))
        if key not in {r[0] for r in results}:
            results.append((key, small))
    return [r[1] for r in results]


def gbs_default_candidates(tuner_cfg):
    """Candidates for the global-batch-size search: the parallel shape is fixed to the best known one and only the
    batch grows (powers of two from the current value up to ``max_search_gbs``)."""
    cand = default_candidates(tuner_cfg)
    gbs = tuner_cfg.get("model_cfg", {}).get("global_batch_size", 1)
    hi = tuner_cfg.get("search_algo", {}).get("max_search_gbs", gbs * 16) if isinstance(tuner_cfg.get("search_algo"), dict) else gbs * 16
    sizes = []
    g = gbs
    while g <= hi:
        sizes.append(g)
        g *= 2
    cand["global_batch_size"] = sizes
    return cand


def gbs_search_all(tuner_cfg):
    cand = gbs_default_candidates(tuner_cfg)
    base = search_all({**tuner_cfg, "candidates": {k: v for k, v in cand.items() if k != "global_batch_size"}})
    out = []
    for gbs in cand["global_batch_size"]:
        for cfg in base:
            c = dict(cfg)
            c["global_batch_size"] = gbs
            c["acc_steps"] = max(1, gbs // (c["dp_degree"] * c["sharding_degree"] * c["micro_batch_size"]))
            if gbs % (c["dp_degree"] * c["sharding_degree"] * c["micro_batch_size"]) == 0:
                out.append(c)
    return out


def add_overlap_performance(cur_cfg, tuner_cfg, history_cfgs):
    """Credit a data-parallel-estimated run with the overlap of gradient all-reduce and backward: the estimate of the
    full job is the small job's throughput times dp, times a measured or configured overlap factor (default 1)."""
    factor = tuner_cfg.get("dp_overlap_factor", 1.0)
    metric = tuner_cfg.get("metric_cfg", {}).get("name", "tokens_per_second")
    if cur_cfg.get(metric) is not None and "estimated_dp_degree" in cur_cfg:
        cur_cfg[f"bw_{metric}"] = cur_cfg[metric] * cur_cfg["estimated_dp_degree"] * factor
    return cur_cfg


# ------------------------------------------------------------------------------------------------ launcher arguments
def _set_path(d, path, value):
    cur = d
    parts = path.split(".")
    for p in parts[:-1]:
        cur = cur.setdefault(p, {})
    cur[parts[-1]] = value


def gen_new_args(raw_args, cfg, tuner_cfg, run_best=False):
    """Command line of the next trial: ``raw_args`` with every tuned key injected in the form the training script
    declares under ``tuner_cfg["run_cmd"]``.  Each entry maps a key to either ``["-o", "Distributed.dp_degree"]``
    (appends ``-o Distributed.dp_degree=2``), ``["--dp_degree"]`` (appends ``--dp_degree 2``) or
    ``["config.json", "a.b.c"]`` (rewrites that key of a JSON / YAML file next to the original, suffixed with the
    trial's shape, and substitutes the new path in the arguments)."""
    import json
    res = list(copy.deepcopy(raw_args))
    run_cmd = tuner_cfg.get("run_cmd", {})
    rewritten = {}
    derived = dict(cfg)
    if "global_batch_size" in cfg and "micro_batch_size" in cfg:
        dpsh = cfg.get("dp_degree", 1) * cfg.get("sharding_degree", 1)
        derived.setdefault("local_batch_size", cfg["global_batch_size"] // dpsh)
        derived.setdefault("gradient_accumulation_steps", max(1, cfg["global_batch_size"] // dpsh // cfg["micro_batch_size"]))
    if run_best and "search_algo" in run_cmd:
        run_cmd = {k: v for k, v in run_cmd.items() if k != "search_algo"}
    for key, spec in run_cmd.items():
        if key not in derived or not isinstance(spec, (list, tuple)) or not spec:
            continue
        val = derived[key]
        if len(spec) == 2 and spec[0] in ("-o", "--override"):
            res += [spec[0], f"{spec[1]}={val}"]
        elif len(spec) == 1:
            if isinstance(val, bool) and tuner_cfg.get("bool_flags_as_switch"):
                if val:
                    res.append(spec[0])
            else:
                res += [spec[0], str(val)]
        elif len(spec) == 2 and spec[0].endswith((".json", ".yaml", ".yml")):
            rewritten.setdefault(spec[0], []).append((spec[1], val))
        elif len(spec) >= 2:
            res += [spec[0], f"{spec[1]}={val}"]
    for path, edits in rewritten.items():
        if path.endswith(".json"):
            with open(path) as f:
                doc = json.load(f)
        else:
            import yaml
            with open(path) as f:
                doc = yaml.safe_load(f)
        for dotted, val in edits:
            _set_path(doc, dotted, val)
        tag = "_".join(f"{k.split('_')[0]}{cfg[k]}" for k in ("dp_degree", "mp_degree", "pp_degree", "sharding_degree",
                                                               "micro_batch_size") if k in cfg)
        stem, ext = os.path.splitext(path)
        new_path = f"{stem}_{tag}{ext}"
        with open(new_path, "w") as f:
            if ext == ".json":
                json.dump(doc, f, indent=2)
            else:
                import yaml
                yaml.safe_dump(doc, f)
        res = [new_path if a == path else a for a in res]
    return res


def gen_sharding_overlap_args(res_args, cfg, tuner_cfg):
    """Extra switches for sharded runs (communication overlap), taken from ``tuner_cfg["sharding_overlap"]``."""
    extra = tuner_cfg.get("sharding_overlap")
    if extra and cfg.get("sharding_degree", 1) > 1:
        res_args = list(res_args) + list(extra if isinstance(extra, (list, tuple)) else [extra])
    return res_args


# ------------------------------------------------------------------------------------------------------- log reading
_OOM_PATTERNS = ("out of memory", "CUDA out of memory", "OutOfMemoryError", "ResourceExhaustedError", "cudaErrorMemoryAllocation")


def _worker_logs(path, file_pattern):
    if os.path.isfile(path):
        return [path]
    if not os.path.isdir(path):
        return []
    rx = re.compile(file_pattern)
    return sorted(os.path.join(path, f) for f in os.listdir(path) if rx.search(f))


def read_metric_log(path, file="workerlog(\\.\\d+)?", target_metric="ips"):
    """``(value, error flag)`` from the newest matching log: the mean of the metric over the recorded steps after
    dropping the first ones (warm-up) - the last 10 at most.  Flags: 0 ok, 1 metric absent, 2 file absent."""
    logs = _worker_logs(path, file)
    if not logs:
        return 0.0, 2
    rx = re.compile(re.escape(target_metric) + r"\s*[:=]\s*([-+]?\d+(?:\.\d+)?(?:[eE][-+]?\d+)?)")
    best = None
    for log in logs:
        with open(log, errors="replace") as f:
            vals = [float(m.group(1)) for line in f for m in rx.finditer(line)]
        if vals:
            best = vals
            break
    if not best:
        return 0.0, 1
    tail = best[len(best) // 5:] if len(best) >= 5 else best
    tail = tail[-10:]
    return round(sum(tail) / len(tail), 5), 0


def read_step_time_log(path, file="workerlog(\\.\\d+)?", target_metric="interval_runtime"):
    return read_metric_log(path, file, target_metric)


def read_allocated_memory_log(path, file="workerlog(\\.\\d+)?", target_metric="max_memory_allocated"):
    logs = _worker_logs(path, file)
    if not logs:
        return 0.0, 2
    rx = re.compile(re.escape(target_metric) + r"\s*[:=]\s*(\d+(?:\.\d+)?)")
    peak = None
    for log in logs:
        with open(log, errors="replace") as f:
            for line in f:
                for m in rx.finditer(line):
                    peak = max(peak or 0.0, float(m.group(1)))
    return (peak, 0) if peak is not None else (0.0, 1)


def read_memory_log(path, file):
    """``(peak MiB, flag)`` from a CSV written by a GPU memory sampler (column ``memory.used`` or ``used``)."""
    target = os.path.join(path, file) if os.path.isdir(path) else path
    if not os.path.exists(target):
        return 0.0, 2
    peak = None
    with open(target) as f:
        for row in csv.DictReader(f):
            for k, v in row.items():
                if k and "used" in k.lower():
                    try:
                        num = float(re.sub(r"[^\d.]", "", v))
                    except ValueError:
                        continue
                    peak = max(peak or 0.0, num)
    return (peak, 0) if peak is not None else (0.0, 1)


def read_completed(path):
    """True when any worker log carries the ``training completed`` marker of the trainer."""
    for log in _worker_logs(path, "workerlog(\\.\\d+)?"):
        with open(log, errors="replace") as f:
            if any("completed" in line.lower() and "train" in line.lower() for line in f):
                return True
    return False


def find_error_from_log(path, file="workerlog(\\.\\d+)?"):
    """0: no error, 1: out of memory, 2: another error (a Python traceback or a fatal signal)."""
    code = 0
    for log in _worker_logs(path, file):
        with open(log, errors="replace") as f:
            text = f.read()
        low = text.lower()
        if any(p.lower() in low for p in _OOM_PATTERNS):
            return 1
        if "traceback (most recent call last)" in low or "segmentation fault" in low or "fatal" in low:
            code = 2
    return code


def read_log(path, metric_file="workerlog.0", target_metric="ips", memory_file=None):
    """Everything the tuner records about a finished trial, as a dict of values and error flags."""
    out = {}
    val, flag = read_metric_log(path, metric_file, target_metric)
    out[target_metric] = val if flag == 0 else None
    out["metric_flag"] = flag
    if memory_file:
        mem, mflag = read_memory_log(path, memory_file)
    else:
        mem, mflag = read_allocated_memory_log(path)
    out["max_mem_usage"] = mem if mflag == 0 else None
    out["memory_flag"] = mflag
    err = find_error_from_log(path)
    out["error_info"] = {0: None, 1: "OOM", 2: "Error"}[err]
    if err == 1:
        out["max_mem_usage"] = "OOM"
    return out


def load_configs_from_csv(configs_csv):
    """Rows of a user-written CSV as configuration dicts (numbers and booleans converted) - for ``CustomizeSearch``."""
    out = []
    with open(configs_csv) as f:
        for row in csv.DictReader(f):
            cfg = {}
            for k, v in row.items():
                v = v.strip() if isinstance(v, str) else v
                if v in ("", None):
                    continue
                if v.lower() in ("true", "false"):
                    cfg[k] = v.lower() == "true"
                else:
                    try:
                        cfg[k] = int(v)
                    except ValueError:
                        try:
                            cfg[k] = float(v)
                        except ValueError:
                            cfg[k] = v
            out.append(cfg)
    return out


def memory_sort(cfg):
    """Sort key: configurations expected to need LESS memory first (more model sharding, smaller micro-batch,
    recompute on)."""
    return (-cfg.get("mp_degree", 1) * cfg.get("pp_degree", 1), -cfg.get("sharding_degree", 1) * cfg.get("sharding_stage", 1),
            cfg.get("micro_batch_size", 1), not cfg.get("use_recompute", False))


def performance_sort(cfg):
    """Sort key: configurations expected to run FASTER first."""
    return (cfg.get("pp_degree", 1), cfg.get("mp_degree", 1), -cfg.get("micro_batch_size", 1), bool(cfg.get("use_recompute")))


def sort_by_special(cfgs, tuner_cfg):
    """Order a candidate list by the strategy named in ``tuner_cfg["search_algo"]["sort"]`` (``memory`` or
    ``performance``, the default)."""
    algo = tuner_cfg.get("search_algo", {})
    how = algo.get("sort", "performance") if isinstance(algo, dict) else "performance"
    if how == "estimated":
        return sort_by_estimated_time(cfgs, tuner_cfg)
    return sorted(cfgs, key=memory_sort if how == "memory" else performance_sort)


def sort_by_estimated_time(cfgs, tuner_cfg):
    """Order by the analytic step-time estimate of ``paddle.cost_model.analytic`` (fastest first); configurations the
    estimate puts above the memory limit are dropped.  Needs the model description in ``tuner_cfg["model_cfg"]``."""
    from ...cost_model.analytic import rank_configs
    return rank_configs(tuner_cfg["model_cfg"], cfgs, memory_limit_gb=tuner_cfg.get("max_mem_usage"))
