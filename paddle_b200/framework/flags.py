"""Global flag registry (paddle/common/flags.cc; ``paddle.set_flags/get_flags``,
python/paddle/base/framework.py:132,157).  Flags are initialised from ``FLAGS_<name>`` environment
variables at import and mirrored into the native runtime when it is loaded, so C++ code reads the same
values."""
from __future__ import annotations

import os

_DEFAULTS = {
    "FLAGS_check_nan_inf": False,
    "FLAGS_check_nan_inf_level": 0,
    "FLAGS_benchmark": False,
    "FLAGS_cudnn_deterministic": False,
    "FLAGS_embedding_deterministic": 0,
    "FLAGS_enable_async_trace": False,
    "FLAGS_enable_nccl_dynamic_check": False,
    "FLAGS_eager_communication_connection": False,
    "FLAGS_allocator_strategy": "auto_growth",
    "FLAGS_fraction_of_gpu_memory_to_use": 0.92,
    "FLAGS_use_stream_safe_cuda_allocator": True,
    "FLAGS_flash_attn_version": 2,
    "FLAGS_nccl_nrings": 1,
    "FLAGS_stop_check_timeout": 900,
    "FLAGS_sharding_sort_parameters": True,
    "FLAGS_pp_check_naninf": False,
    "FLAGS_sharding_v2_check_zero_padding": False,
    "FLAGS_shard_bypass_dygraph_optimizer": False,
    "FLAGS_check_kernel_launch": False,
    "FLAGS_sync_after_alloc": False,
    "FLAGS_use_cuda_managed_memory": False,
    "FLAGS_log_memory_stats": False,
    "FLAGS_trace_api": "",
    "FLAGS_pd_wait_limit_ms": 2000,
}
_flags = {}


def _parse(default, raw: str):
    if isinstance(default, bool):
        return raw.lower() in ("1", "true", "yes", "on")
    if isinstance(default, int):
        return int(raw)
    if isinstance(default, float):
        return float(raw)
    return raw


def _init():
    for k, v in _DEFAULTS.items():
        raw = os.environ.get(k)
        _flags[k] = _parse(v, raw) if raw is not None else v


_init()


def _norm(name: str) -> str:
    return name if name.startswith("FLAGS_") else "FLAGS_" + name


def set_flags(flags: dict):
    for k, v in flags.items():
        k = _norm(k)
        if k not in _flags:
            raise ValueError(f"Flag {k} cannot set its value through this function.")
        _flags[k] = v
        _apply_side_effect(k, v)


def get_flags(flags):
    names = [flags] if isinstance(flags, str) else list(flags)
    out = {}
    for k in names:
        k = _norm(k)
        if k not in _flags:
            raise ValueError(f"Flag {k} cannot get its value through this function.")
        out[k] = _flags[k]
    return out


def flag(name: str):
    return _flags[_norm(name)]


def _apply_side_effect(k, v):
    import torch
    if k == "FLAGS_cudnn_deterministic":
        torch.backends.cudnn.deterministic = bool(v)
    elif k == "FLAGS_check_nan_inf":
        from ..amp import debugging
        (debugging.enable_tensor_checker if v else debugging.disable_tensor_checker)()
