"""Auto-tuner mode of the launcher (``--auto_tuner_json``; python/paddle/distributed/launch/main.py:300-1100): run the
training script once per candidate configuration, each trial in its own log directory with the tuned values injected
into its command line, read throughput / memory / errors back from the worker logs, record every trial in a CSV that
an interrupted search resumes from, and finally (optionally) run the best configuration for real."""
from __future__ import annotations

import copy
import json
import os
import sys
import time


def _load_cfg(path):
    with open(path) as f:
        if path.endswith((".yaml", ".yml")):
            import yaml
            return yaml.safe_load(f)
        return json.load(f)


def _trial_name(cfg):
    short = (("dp_degree", "DP"), ("mp_degree", "MP"), ("pp_degree", "PP"), ("vpp_degree", "VPP"), ("sharding_degree", "Sharding"),
             ("sharding_stage", "Stage"), ("micro_batch_size", "MBS"), ("use_recompute", "Recompute"), ("global_batch_size", "GBS"))
    return "_".join(f"{s}{cfg[k]}" for k, s in short if cfg.get(k) is not None)


def _run_trial(args, script_args, log_dir, timeout, nproc=None):
    """One pod run with its own log directory; returns (exit code, seconds, timed out)."""
    from .main import CollectiveController
    a = copy.copy(args)
    a.training_script_args = list(script_args)
    a.log_dir = log_dir
    a.elastic_level = -1
    a.max_restart = 0
    if nproc is not None:
        a.nproc_per_node = nproc
        a.devices = None
    ctl = CollectiveController(a)
    t0 = time.time()
    ctl.build_pod()
    ctl.pod.deploy()
    timed_out = False
    while True:
        st = ctl.pod.status()
        if st != "RUNNING":
            break
        if timeout and time.time() - t0 > timeout:
            timed_out = True
            break
        time.sleep(a.poll_interval)
    failed = ctl.pod.failed()
    ctl.pod.stop()
    code = 0 if st == "COMPLETED" else (failed[0][1].poll() if failed else 1)
    return code, time.time() - t0, timed_out


def run_auto_tuner(args):
    """Returns the process exit code.  ``args`` are the launcher's parsed arguments (``auto_tuner_json`` set)."""
    from ..auto_tuner import AutoTuner
    from ..auto_tuner.utils import add_overlap_performance, gen_new_args, read_log
    tuner_cfg = _load_cfg(args.auto_tuner_json)
    nnodes = int(str(args.nnodes).split(":")[0])
    ctl_devices = args.nproc_per_node
    if ctl_devices is None:
        from .main import CollectiveController
        ctl_devices = len(CollectiveController(args)._local_devices())
    tuner_cfg.setdefault("nodes", nnodes)
    tuner_cfg.setdefault("gpus_per_node", ctl_devices)
    tuner_cfg.setdefault("num_gpus", nnodes * ctl_devices)
    metric = tuner_cfg.setdefault("metric_cfg", {}).setdefault("name", "ips")
    tuner_cfg["metric_cfg"].setdefault("OptimizationDirection", "max")
    root = args.log_dir
    os.makedirs(root, exist_ok=True)
    history_csv = os.path.join(root, f"{args.job_id}_history.csv")
    tuner = AutoTuner(tuner_cfg)
    if tuner.resume_form_history(history_csv):
        sys.stderr.write(f"[auto_tuner] resumed {len(tuner.resume_cfgs)} finished trials from {history_csv}\n")
    timeout = tuner_cfg.get("max_time_per_task")
    raw_args = list(args.training_script_args)
    job = 0
    while True:
        cfg = tuner.search_once()
        if cfg is None:
            break
        job += 1
        cfg = dict(cfg)
        name = _trial_name(cfg)
        log_dir = os.path.join(root, name)
        trial_args = gen_new_args(raw_args, cfg, tuner_cfg)
        sys.stderr.write(f"[auto_tuner] trial {job}: {name}\n")
        nproc = None
        if "num_gpus" in cfg and cfg["num_gpus"] != tuner_cfg["num_gpus"]:      # data-parallel estimation: a smaller job
            nproc = max(1, cfg["num_gpus"] // nnodes)
        code, secs, timed_out = _run_trial(args, trial_args, log_dir, timeout, nproc)
        res = read_log(log_dir, "workerlog(\\.\\d+)?", metric, tuner_cfg.get("memory_file"))
        cfg.update(job_id=job, exec_time=round(secs, 2), **res)
        if timed_out and cfg.get(metric) is None:
            cfg["error_info"] = cfg["error_info"] or "Timeout"
        elif code != 0 and not cfg["error_info"]:
            cfg["error_info"] = "Error"
        if cfg["error_info"]:
            cfg[metric] = None
        add_overlap_performance(cfg, tuner_cfg, tuner.history_cfgs)
        tuner.add_cfg(cfg)
        tuner.store_history(history_csv)
    best = tuner.get_best()
    if best is None:
        sys.stderr.write("[auto_tuner] no configuration ran to completion\n")
        return 1
    with open(os.path.join(root, f"{args.job_id}_best_cfg.json"), "w") as f:
        json.dump(best, f, indent=2, default=str)
    sys.stderr.write(f"[auto_tuner] best: {_trial_name(best)} {metric}={best.get(metric)}\n")
    if tuner_cfg.get("run_best", False):
        code, _, _ = _run_trial(args, gen_new_args(raw_args, best, tuner_cfg, run_best=True), os.path.join(root, "best_cfg"), None)
        return code
    return 0
