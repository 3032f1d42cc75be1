"""``paddle.incubate``: fused layers / operators, MoE, extra optimizers, graph and segment helpers."""
from __future__ import annotations

import importlib

from . import nn  # noqa: F401


def __getattr__(name):
    if name in ("distributed", "optimizer", "autograd", "asp", "tensor", "operators", "framework", "multiprocessing",
                "passes", "xpu", "jit", "layers", "autotune"):
        return importlib.import_module(f"{__name__}.{name}")
    if name == "inference":
        from .jit import inference
        return inference
    if name in ("LookAhead", "ModelAverage"):
        from . import optimizer
        return getattr(optimizer, name)
    if name in ("segment_sum", "segment_mean", "segment_max", "segment_min", "graph_send_recv", "graph_reindex",
                "graph_sample_neighbors", "graph_khop_sampler", "softmax_mask_fuse", "softmax_mask_fuse_upper_triangle",
                "identity_loss"):
        from . import operators
        return getattr(operators, name)
    raise AttributeError(name)
