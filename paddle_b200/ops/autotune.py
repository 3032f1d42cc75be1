"""Run-time kernel configuration cache (reference: the algorithm cache of paddle/phi/kernels/autotune/ and
``paddle.incubate.autotune.set_config``).

The tunable launches of this framework have one integer knob each (K splits of the skinny decode GEMM, context
splits of the paged decode attention, ...).  While tuning is enabled and the step counter is inside the tuning
range, the first call of an ``(op, key)`` pair times every candidate with CUDA events and stores the fastest; later
calls (and all calls outside the range) read the cache, falling back to the built-in heuristic on a miss.  The cache
can be saved to / loaded from JSON so that a serving process starts tuned."""
from __future__ import annotations

import json
import threading

_lock = threading.Lock()
_cache = {}                       # (op, key tuple) -> chosen candidate
_stats = {"hit": 0, "miss": 0, "tuned": 0}
_cfg = {"enable": False, "tuning_range": (1, 10)}
_step = 0


def set_kernel_config(enable=None, tuning_range=None):
    if enable is not None:
        _cfg["enable"] = bool(enable)
    if tuning_range is not None:
        lo, hi = tuning_range
        _cfg["tuning_range"] = (int(lo), int(hi))


def step():
    """Called once per training / decode step by the optimizers and the decode engine."""
    global _step
    _step += 1


def tuning_now():
    lo, hi = _cfg["tuning_range"]
    return _cfg["enable"] and lo <= max(_step, 1) <= hi


def status():
    total = _stats["hit"] + _stats["miss"]
    return {"step": _step, "use_autotune": tuning_now(), "cache_size": len(_cache),
            "cache_hit_rate": (_stats["hit"] / total) if total else 0.0, "tuned": _stats["tuned"]}


def _default_timer(fn, iters=3):
    import torch
    fn()                                            # warm-up, also loads the kernel
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / iters


def choose(op, key, candidates, run, default, timer=None):
    """Returns the configuration to use for ``(op, key)``.  ``run(candidate)`` launches the kernel once with that
    candidate (it must be safe to repeat: outputs are overwritten, accumulators restored by the caller)."""
    k = (op, tuple(key))
    with _lock:
        got = _cache.get(k)
    if got is not None:
        _stats["hit"] += 1
        return got
    _stats["miss"] += 1
    if not tuning_now():
        return default
    import torch
    if timer is None and (not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing()):
        return default
    timer = timer or _default_timer
    best, best_t = default, float("inf")
    for c in candidates:
        try:
            t = timer(lambda c=c: run(c))
        except Exception:
            continue
        if t < best_t:
            best, best_t = c, t
    with _lock:
        _cache[k] = best
    _stats["tuned"] += 1
    return best


def save(path):
    with _lock:
        data = [{"op": op, "key": list(key), "choice": v} for (op, key), v in _cache.items()]
    with open(path, "w") as f:
        json.dump(data, f)


def load(path):
    with open(path) as f:
        data = json.load(f)
    with _lock:
        for d in data:
            _cache[(d["op"], tuple(d["key"]))] = d["choice"]
    return len(data)


def clear():
    global _step
    with _lock:
        _cache.clear()
    _stats.update(hit=0, miss=0, tuned=0)
    _step = 0
