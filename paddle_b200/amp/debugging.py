"""Numerics debugging (python/paddle/amp/debugging.py): nan/inf checks and per-dtype operator
statistics gathered through a torch dispatch mode."""
from __future__ import annotations

import collections
import contextlib

import torch
from torch.utils._python_dispatch import TorchDispatchMode


class DebugMode:
    CHECK_NAN_INF_AND_ABORT = 0
    CHECK_NAN_INF = 1
    CHECK_ALL_FOR_OVERFLOW = 2
    CHECK_ALL = 4


def check_numerics(tensor, op_type="", var_name="", debug_mode=DebugMode.CHECK_NAN_INF_AND_ABORT):
    t = tensor.detach().float()
    n_nan, n_inf = int(torch.isnan(t).sum()), int(torch.isinf(t).sum())
    if (n_nan or n_inf) and debug_mode == DebugMode.CHECK_NAN_INF_AND_ABORT:
        raise RuntimeError(f"[check_numerics] op={op_type} var={var_name}: {n_nan} nan, {n_inf} inf")
    stats = torch.tensor([n_nan, n_inf, int((t == 0).sum())], dtype=torch.int64)
    vals = torch.stack([t.max(), t.min(), t.mean()]) if t.numel() else torch.zeros(3)
    return stats, vals


class _NanInfMode(TorchDispatchMode):
    """Checks every operator output.  ``CHECK_NAN_INF_AND_ABORT`` raises at the first NaN / Inf; the other modes print
    one line per offending operator and go on; ``checked_op_list`` / ``skipped_op_list`` filter by operator name."""

    def __init__(self, config=None):
        super().__init__()
        self.debug_mode = getattr(config, "debug_mode", DebugMode.CHECK_NAN_INF_AND_ABORT)
        self.checked = set(getattr(config, "checked_op_list", None) or [])
        self.skipped = set(getattr(config, "skipped_op_list", None) or [])
        self.found = []

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        name = str(getattr(func, "overloadpacket", func)).split(".")[-1]
        if (self.checked and name not in self.checked) or name in self.skipped:
            return out
        for o in (out if isinstance(out, (tuple, list)) else (out,)):
            if isinstance(o, torch.Tensor) and o.is_floating_point() and o.numel() and not bool(torch.isfinite(o).all()):
                if self.debug_mode == DebugMode.CHECK_NAN_INF_AND_ABORT:
                    raise RuntimeError(f"nan/inf produced by {func}")
                n_nan, n_inf = int(torch.isnan(o).sum()), int(torch.isinf(o).sum())
                self.found.append((name, n_nan, n_inf))
                print(f"[tensor checker] {func}: {n_nan} nan, {n_inf} inf in an output of shape {list(o.shape)}")
        return out


class _OpStatsMode(TorchDispatchMode):
    def __init__(self):
        super().__init__()
        self.stats = collections.defaultdict(lambda: collections.Counter())

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        o = out[0] if isinstance(out, (tuple, list)) and out else out
        if isinstance(o, torch.Tensor):
            self.stats[str(func.overloadpacket)][str(o.dtype).replace("torch.", "")] += 1
        return out


_modes = {}


def enable_tensor_checker(checker_config=None):
    if checker_config is not None and not getattr(checker_config, "enable", True):
        return
    disable_tensor_checker()
    m = _NanInfMode(checker_config)
    m.__enter__()
    _modes["nan"] = m


def disable_tensor_checker():
    m = _modes.pop("nan", None)
    if m is not None:
        m.__exit__(None, None, None)


class TensorCheckerConfig:
    def __init__(self, enable=True, debug_mode=DebugMode.CHECK_NAN_INF_AND_ABORT, output_dir=None,
                 checked_op_list=None, skipped_op_list=None, debug_step=None, stack_height_limit=1):
        self.enable, self.debug_mode = enable, debug_mode
        self.output_dir, self.checked_op_list, self.skipped_op_list = output_dir, checked_op_list, skipped_op_list
        self.debug_step, self.stack_height_limit = debug_step, stack_height_limit


def enable_operator_stats_collection():
    m = _OpStatsMode()
    m.__enter__()
    _modes["ops"] = m


def disable_operator_stats_collection():
    m = _modes.pop("ops", None)
    if m is None:
        return {}
    m.__exit__(None, None, None)
    print("<------------------------------ op list ------------------------------>")
    for op, c in sorted(m.stats.items()):
        print(f"  {op:50s} fp16={c['float16']} bf16={c['bfloat16']} fp32={c['float32']} other="
              f"{sum(v for k, v in c.items() if k not in ('float16', 'bfloat16', 'float32'))}")
    return {k: dict(v) for k, v in m.stats.items()}


@contextlib.contextmanager
def collect_operator_stats():
    enable_operator_stats_collection()
    try:
        yield
    finally:
        disable_operator_stats_collection()


def compare_accuracy(dump_path, another_dump_path, output_filename, loss_scale=1, dump_all_tensors=False):
    raise NotImplementedError("compare_accuracy works on dump files produced by the reference's C++ checker")


def check_layer_numerics(func):
    """Decorator for ``Layer.forward``: checks the tensor inputs and outputs of the call for NaN / Inf and raises with
    the layer's name when one is found (python/paddle/amp/debugging.py ``check_layer_numerics``)."""
    import functools

    import torch

    def scan(where, owner, values):
        for i, v in enumerate(values):
            if isinstance(v, torch.Tensor) and v.is_floating_point():
                t = v.as_subclass(torch.Tensor)
                n_nan, n_inf = int(torch.isnan(t).sum()), int(torch.isinf(t).sum())
                if n_nan or n_inf:
                    raise RuntimeError(f"[PRECISION] [ERROR] in [layer={type(owner).__name__}, {where}={i}, "
                                       f"dtype={t.dtype}], numel={t.numel()}, num_nan={n_nan}, num_inf={n_inf}")

    @functools.wraps(func)
    def wrapper(self, *args, **kwargs):
        if args and not isinstance(args[0], torch.Tensor):
            raise RuntimeError("First input of this layer must be tensor.")
        scan("input", self, args)
        out = func(self, *args, **kwargs)
        scan("output", self, out if isinstance(out, (list, tuple)) else [out])
        return out
    return wrapper
