"""``paddle.incubate.jit.inference`` (python/paddle/incubate/jit/inference_decorator.py): decorator that turns a
layer's forward (or a function) into an inference engine call.  The reference exports the function to a static
program and runs it through the analysis predictor; here the function runs under ``no_grad`` in the requested
precision and, on a GPU, is replayed from a CUDA graph per input signature."""
from __future__ import annotations

import functools

import torch

__all__ = ["inference"]


def inference(function=None, cache_static_model=False, save_model_dir=None, memory_pool_init_size_mb=1000,
              precision_mode="float32", switch_ir_optim=True, switch_ir_debug=False, enable_cinn=False, with_trt=False,
              trt_precision_mode="float32", trt_use_static=False, collect_shape=False, enable_new_ir=True,
              exp_enable_use_cutlass=False, delete_pass_lists=None, skip_prune_program=False, use_cuda_graph=True):
    dtype = {"float32": None, "float16": torch.float16, "bfloat16": torch.bfloat16}.get(precision_mode)
    if precision_mode not in ("float32", "float16", "bfloat16"):
        raise ValueError(f"precision_mode must be float32 / float16 / bfloat16, got {precision_mode}")

    def decorate(fn):
        from ...nn.layer.layers import Layer
        layer = fn if isinstance(fn, Layer) else None
        target = layer.forward if layer is not None else fn
        graphed = {}

        @functools.wraps(target)
        def run(*args, **kwargs):
            def call(*a):
                with torch.no_grad():
                    if dtype is not None and torch.cuda.is_available():
                        with torch.autocast("cuda", dtype=dtype):
                            return target(*a, **kwargs)
                    return target(*a, **kwargs)
            tensors_only = all(isinstance(a, torch.Tensor) for a in args)
            if use_cuda_graph and not kwargs and tensors_only and args and args[0].is_cuda:
                from ...device.cuda.graphs import wrap_cuda_graph
                key = id(target)
                if key not in graphed:
                    graphed[key] = wrap_cuda_graph(call)
                return graphed[key](*args)
            return call(*args)
        if layer is not None:
            layer.__dict__["forward"] = run
            return layer
        return run
    if function is not None:
        return decorate(function)
    return decorate
