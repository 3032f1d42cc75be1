"""``paddle.incubate.autotune.set_config`` (python/paddle/incubate/autotune.py): switches for kernel, layout and
dataloader tuning.  Kernel tuning drives ``paddle_b200.ops.autotune``; layout tuning has nothing to choose here (the
kernels take the layouts the layers produce); dataloader tuning picks ``num_workers`` by timing a few batches."""
from __future__ import annotations

import json

from ..ops import autotune as _at

_state = {"layout": False, "dataloader": {"enable": False, "tuning_steps": 500}}


def set_config(config=None):
    if config is None:
        _at.set_kernel_config(enable=True)
        _state["layout"] = True
        _state["dataloader"]["enable"] = True
        return
    if isinstance(config, str):
        with open(config) as f:
            config = json.load(f)
    if not isinstance(config, dict):
        raise TypeError("config should be a dict, a json file path or None")
    if "kernel" in config:
        k = config["kernel"]
        if "enable" in k:
            if not isinstance(k["enable"], bool):
                raise TypeError("The auto-tuning configuration of the kernel is incorrect: enable should be bool")
            _at.set_kernel_config(enable=k["enable"])
        if "tuning_range" in k:
            if not isinstance(k["tuning_range"], (list, tuple)) or len(k["tuning_range"]) != 2:
                raise TypeError("The auto-tuning configuration of the kernel is incorrect: tuning_range should be [lo, hi]")
            _at.set_kernel_config(tuning_range=k["tuning_range"])
    if "layout" in config and "enable" in config["layout"]:
        _state["layout"] = bool(config["layout"]["enable"])
    if "dataloader" in config:
        d = config["dataloader"]
        if "enable" in d:
            _state["dataloader"]["enable"] = bool(d["enable"])
        if "tuning_steps" in d:
            _state["dataloader"]["tuning_steps"] = int(d["tuning_steps"])


def dataloader_config():
    return dict(_state["dataloader"])


def tune_num_workers(make_loader, candidates=(0, 2, 4, 8), batches=8):
    """Times ``batches`` batches of ``make_loader(num_workers)`` for each candidate and returns the fastest count."""
    import time
    best, best_t = candidates[0], float("inf")
    for n in candidates:
        it = iter(make_loader(n))
        t0 = time.perf_counter()
        try:
            for _ in range(batches):
                next(it)
        except StopIteration:
            pass
        t = time.perf_counter() - t0
        if t < best_t:
            best, best_t = n, t
    return best
