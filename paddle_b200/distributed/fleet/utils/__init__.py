from . import hybrid_parallel_util, mix_precision_utils  # noqa: F401


def __getattr__(name):
    import importlib
    if name in ("sequence_parallel_utils", "tensor_fusion_helper", "timer_helper", "log_util", "fs",
                "tensor_parallel_utils", "pp_parallel_adaptor", "hybrid_parallel_inference"):
        return importlib.import_module(f"{__name__}.{name}")
    if name == "recompute":
        from ..recompute import recompute
        return recompute
    if name in ("LocalFS", "HDFSClient"):
        from . import fs
        return getattr(fs, name)
    raise AttributeError(name)
