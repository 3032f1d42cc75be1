"""API call tracer (python/paddle/api_tracer/api_tracer.py; switched on by ``FLAGS_trace_api``): wraps the public
callables named in a config and appends one line per call (name, argument shapes / dtypes, output shapes) to a file."""
from __future__ import annotations

import functools
import importlib
import threading

__all__ = ["start_api_tracer", "stop_api_tracer"]

_lock = threading.Lock()
_state = {"file": None, "patched": []}


def _describe(v):
    if hasattr(v, "shape") and hasattr(v, "dtype"):
        return f"Tensor(shape={list(v.shape)}, dtype={str(v.dtype).replace('torch.', '')})"
    if isinstance(v, (list, tuple)):
        return type(v).__name__ + "[" + ", ".join(_describe(x) for x in v[:8]) + "]"
    return repr(v)[:60]


def _wrap(name, fn):
    @functools.wraps(fn)
    def traced(*a, **k):
        out = fn(*a, **k)
        f = _state["file"]
        if f is not None:
            args = ", ".join([_describe(x) for x in a] + [f"{key}={_describe(v)}" for key, v in k.items()])
            with _lock:
                f.write(f"{name}({args}) -> {_describe(out)}\n")
                f.flush()
        return out
    traced.__wrapped_api__ = fn
    return traced


def start_api_tracer(api_path, save_config_path):
    """``api_path``: a text file with one dotted API name per line (``paddle.nn.functional.relu``; ``paddle`` names this
    package) or a list of such names; ``save_config_path``: the trace file."""
    stop_api_tracer()
    names = api_path if isinstance(api_path, (list, tuple)) else [ln.strip() for ln in open(api_path) if ln.strip()]
    _state["file"] = open(save_config_path, "a")
    root = __name__.split(".")[0]
    for full in names:
        parts = full.split(".")
        if parts[0] == "paddle":
            parts[0] = root
        mod = importlib.import_module(parts[0])
        for p in parts[1:-1]:
            mod = getattr(mod, p)
        fn = getattr(mod, parts[-1], None)
        if callable(fn) and not hasattr(fn, "__wrapped_api__"):
            setattr(mod, parts[-1], _wrap(full, fn))
            _state["patched"].append((mod, parts[-1], fn))


def stop_api_tracer():
    for mod, attr, fn in _state["patched"]:
        setattr(mod, attr, fn)
    _state["patched"] = []
    if _state["file"] is not None:
        _state["file"].close()
        _state["file"] = None
