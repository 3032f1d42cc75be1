"""Global flag registry (paddle/common/flags.cc; ``paddle.set_flags/get_flags``,
python/paddle/base/framework.py:132,157).  Every flag the reference exports is registered with its type and default,
initialised from the ``FLAGS_<name>`` environment variable at import, and mirrored into the native runtime once that
library is loaded, so C++ code reads the same values.

Each flag is one of three kinds, reported by ``flag_info``:

* ``effect``   - setting it changes behaviour here (the handler is named in the table below);
* ``read``     - consulted where it is used (``flag(name)`` call sites in this package);
* ``inert``    - accepted so that scripts written for the reference keep running, with the reason it changes nothing
                 (the subsystem is supplied by torch, or is a back end that is not built)."""
from __future__ import annotations

import os

_TORCH_ALLOC = "memory comes from torch's caching allocator"
_NO_PS = "parameter-server / GPU-graph engine is not built"
_NO_CINN = "the CINN compiler is not built; hot paths are hand-written kernels and CUDA graphs"
_NO_PIR = "programs are recorded and replayed; there is no PIR interpreter to configure"
_NO_ONEDNN = "CPU vendor libraries are not a target"
_NO_TRT = "TensorRT is not a target"
_DLOPEN = "libraries are located by torch and by the in-tree loader"
_LIBRARY = "library GEMMs and convolutions go through torch's cuBLAS / cuDNN handles"

# name: (default, kind, note)
_SPEC = {
    # numerics / debugging
    "check_nan_inf": (False, "effect", "tensor checker of paddle.amp.debugging"),
    "check_nan_inf_level": (0, "read", "level handed to the tensor checker when FLAGS_check_nan_inf switches it on"),
    "low_precision_op_list": (0, "effect", "operator statistics of paddle.amp.debugging"),
    "call_stack_level": (1, "inert", "Python tracebacks are always complete"),
    "check_kernel_launch": (False, "effect", "synchronise and check the status word after every native launch"),
    "benchmark": (False, "effect", "synchronise after every native launch"),
    "enable_api_kernel_fallback": (True, "inert", "there is one device; nothing to fall back to"),
    "accuracy_check_atol_fp32": (1e-6, "read", "default tolerances of the accuracy_check operator"),
    "accuracy_check_rtol_fp32": (1e-6, "read", "default tolerances of the accuracy_check operator"),
    "accuracy_check_atol_fp16": (1e-3, "read", "default tolerances of the accuracy_check operator"),
    "accuracy_check_rtol_fp16": (1e-3, "read", "default tolerances of the accuracy_check operator"),
    "accuracy_check_atol_bf16": (1e-3, "read", "default tolerances of the accuracy_check operator"),
    "accuracy_check_rtol_bf16": (1e-3, "read", "default tolerances of the accuracy_check operator"),
    "alloc_fill_value": (-1, "inert", _TORCH_ALLOC),
    "sync_after_alloc": (False, "inert", _TORCH_ALLOC),
    "set_to_1d": (False, "inert", "0-d tensors keep shape []"),
    "sort_sum_gradient": (False, "inert", "gradient accumulation order is torch autograd's"),
    "max_inplace_grad_add": (0, "inert", "gradient accumulation is torch autograd's"),
    # threads
    "paddle_num_threads": (1, "effect", "torch.set_num_threads"),
    "inner_op_parallelism": (0, "effect", "torch.set_num_interop_threads (before the first parallel region only)"),
    "dist_threadpool_size": (0, "inert", _NO_PS),
    # library math
    "enable_cublas_tensor_op_math": (False, "effect", "torch.backends.cuda.matmul.allow_tf32"),
    "gemm_use_half_precision_compute_type": (False, "effect", "reduced-precision reductions of library half GEMMs"),
    "cublaslt_exhaustive_search_times": (0, "inert", _LIBRARY),
    "enable_blaslt_global_search": (False, "inert", _LIBRARY),
    "cublaslt_device_best_config": ("", "inert", _LIBRARY),
    "cuda_core_int8_gemm": (False, "inert", _LIBRARY),
    "cudnn_deterministic": (False, "effect", "torch.backends.cudnn.deterministic"),
    "embedding_deterministic": (0, "effect", "deterministic algorithms (warn only) for scatter-add style gradients"),
    "cudnn_exhaustive_search": (False, "effect", "torch.backends.cudnn.benchmark"),
    "cudnn_exhaustive_search_times": (-1, "inert", _LIBRARY),
    "cudnn_batchnorm_spatial_persistent": (False, "inert", _LIBRARY),
    "batch_norm_use_miopen": (False, "inert", "ROCm is not a target"),
    "conv2d_disable_cudnn": (False, "effect", "torch.backends.cudnn.enabled"),
    "enable_cudnn_frontend": (False, "inert", _LIBRARY),
    "cudnn_cache_saturation_count": (1, "inert", _LIBRARY),
    "manually_trans_conv_filter": (False, "inert", _LIBRARY),
    "use_fast_math": (False, "inert", "kernels are compiled ahead of time with fixed math flags"),
    "einsum_opt": (False, "inert", "einsum is torch's"),
    "use_autotune": (False, "effect", "kernel auto-tuning of paddle_b200.ops.autotune"),
    "search_cache_max_number": (1000000, "inert", "the tuning cache is unbounded and keyed by (op, shape)"),
    "flash_attn_version": (2, "inert", "attention runs the in-tree tcgen05 kernels"),
    "use_xqa_optim": (False, "inert", "decode attention is the in-tree paged kernel"),
    "fused_multi_transformer_op_use_mbfmha": (False, "inert", "decode attention is the in-tree paged kernel"),
    "multi_block_attention_min_partition_size": (1024, "inert", "decode attention picks its own split"),
    # device selection / memory
    "selected_gpus": ("", "read", "device of this rank; exported per rank by the launcher"),
    "allocator_strategy": ("auto_growth", "inert", _TORCH_ALLOC),
    "fraction_of_gpu_memory_to_use": (0.92, "effect", "torch.cuda.set_per_process_memory_fraction"),
    "gpu_memory_limit_mb": (0, "effect", "torch.cuda.set_per_process_memory_fraction from an absolute size"),
    "initial_gpu_memory_in_mb": (0, "inert", _TORCH_ALLOC),
    "reallocate_gpu_memory_in_mb": (0, "inert", _TORCH_ALLOC),
    "auto_growth_chunk_size_in_mb": (0, "inert", _TORCH_ALLOC),
    "fraction_of_cpu_memory_to_use": (1.0, "inert", _TORCH_ALLOC),
    "initial_cpu_memory_in_mb": (500, "inert", _TORCH_ALLOC),
    "fraction_of_cuda_pinned_memory_to_use": (0.5, "inert", _TORCH_ALLOC),
    "use_auto_growth_pinned_allocator": (False, "inert", _TORCH_ALLOC),
    "pinned_memory_as_cpu_backend": (False, "inert", _TORCH_ALLOC),
    "use_cuda_malloc_async_allocator": (False, "effect", "PYTORCH_CUDA_ALLOC_CONF=backend:cudaMallocAsync when set before CUDA starts"),
    "cuda_malloc_async_pool_memory_throttle_ratio": (0.8, "inert", _TORCH_ALLOC),
    "auto_free_cudagraph_allocations_on_launch": (True, "inert", "graph pools are torch's"),
    "use_stream_safe_cuda_allocator": (True, "inert", _TORCH_ALLOC),
    "use_cuda_managed_memory": (False, "inert", _TORCH_ALLOC),
    "eager_delete_tensor_gb": (0.0, "inert", "tensors are freed by reference counting"),
    "fast_eager_deletion_mode": (True, "inert", "tensors are freed by reference counting"),
    "memory_fraction_of_eager_deletion": (1.0, "inert", "tensors are freed by reference counting"),
    "eager_delete_scope": (True, "inert", "there are no scopes"),
    "local_exe_sub_scope_limit": (256.0, "inert", "there are no scopes"),
    "enable_record_memory": (False, "inert", "memory events come from the activity tracer (profile_memory)"),
    "log_memory_stats": (False, "effect", "print the allocator summary at interpreter exit"),
    "use_shm_cache": (False, "inert", "worker processes hand batches over through torch's shared memory"),
    "dataloader_use_file_descriptor": (False, "effect", "torch.multiprocessing sharing strategy"),
    "reader_queue_speed_test_mode": (False, "inert", "no reader queue"),
    # communication
    "sync_nccl_allreduce": (True, "inert", "collectives are ordered by stream events"),
    "nccl_blocking_wait": (False, "inert", "Task.wait / sync_op decide per call whether the host blocks"),
    "benchmark_nccl": (False, "inert", "synchronise explicitly, or time with CUDA events"),
    "eager_communication_connection": (False, "inert", "NCCL communicators are created with the group (device_id is passed at init)"),
    "dynamic_static_unified_comm": (True, "inert", "one communication library for both modes"),
    "enable_async_trace": (False, "read", "init_parallel_env starts the communication watchdog"),
    "async_trace_count": (5, "inert", "the watchdog keeps the last finished collective per group"),
    "enable_nccl_dynamic_check": (False, "read", "shape / dtype exchange before collectives"),
    "allreduce_record_one_event": (False, "inert", "collectives are ordered by stream events"),
    "nccl_nrings": (1, "inert", "channel count is NCCL's choice"),
    "tcp_max_syn_backlog": (2048, "inert", "the TCP store listens with the system's maximum backlog"),
    "get_host_by_name_time": (120, "inert", "rendezvous addresses are numeric"),
    "stop_check_timeout": (900, "inert", "rendezvous waits are bounded by the process-group timeout"),
    "enable_auto_parallel_align_mode": (False, "read", "auto-parallel: accumulate in the reference order for loss alignment"),
    "enable_all2all_use_fp16": (False, "inert", _NO_PS),
    "enable_tracker_all2all": (False, "inert", _NO_PS),
    "enable_sparse_inner_gather": (False, "inert", _NO_PS),
    "enable_auto_detect_gpu_topo": (True, "inert", "every GPU pair is one NVSwitch hop"),
    "enable_auto_rdma_trans": (True, "inert", _NO_PS),
    "communicator_max_merge_var_num": (20, "inert", _NO_PS),
    "communicator_is_sgd_optimizer": (True, "inert", _NO_PS),
    "communicator_send_queue_size": (20, "inert", _NO_PS),
    "enable_exit_when_partial_worker": (False, "inert", _NO_PS),
    # distributed training switches of the Python layer
    "sharding_sort_parameters": (True, "read", "sharding: size-sorted parameter placement"),
    "pp_check_naninf": (False, "read", "pipeline: check activations for NaN / Inf"),
    "sharding_v2_check_zero_padding": (False, "inert", "fused buffers are zero-filled at creation and padding is never written"),
    "shard_bypass_dygraph_optimizer": (False, "inert", "profile with the profiler's model view instead"),
    # programs / executor / compiler
    "new_executor_use_cuda_graph": (False, "inert", "wrap the program in CompiledProgram(..., cuda_graph=True)"),
    "print_ir": (False, "inert", "print(program) shows a recorded program at any time"),
    "prim_enable_dynamic": (False, "inert", "decomposition is requested per program through paddle.decomposition.decompose"),
    "prim_skip_dynamic": (True, "inert", "decomposition is requested per program through paddle.decomposition.decompose"),
    "prim_check_ops": (False, "inert", "is_primitive_program reports what is left after decomposition"),
    "prim_forward_blacklist": ("", "inert", "decompose takes blacklist / whitelist arguments"),
    "apply_pass_to_program": (False, "inert", _NO_PIR),
    "enable_pir_api": (True, "inert", _NO_PIR),
    "enable_pir_in_executor": (False, "inert", _NO_PIR),
    "enable_pir_in_executor_trace_run": (False, "inert", _NO_PIR),
    "enable_pir_with_pt_in_dy2st": (True, "inert", _NO_PIR),
    "pir_apply_inplace_pass": (True, "inert", _NO_PIR),
    "pir_apply_shape_optimization_pass": (False, "inert", _NO_PIR),
    "pir_broadcast_tree_limit": (32, "inert", _NO_PIR),
    "pir_interpreter_record_stream_for_gc_cache": (False, "inert", _NO_PIR),
    "ir_inplace_kernel_blacklist": ("", "inert", _NO_PIR),
    "logging_pir_py_code_dir": ("", "inert", _NO_PIR),
    "logging_pir_py_code_int_tensor_element_limit": (2048, "inert", _NO_PIR),
    "logging_trunc_pir_py_code": (True, "inert", _NO_PIR),
    "logging_pir_py_code_dump_symbolic_dims": (False, "inert", _NO_PIR),
    "check_infer_symbolic": (False, "inert", _NO_PIR),
    "enable_cse_in_dy2st": (True, "inert", _NO_PIR),
    "cse_max_count": (-1, "inert", _NO_PIR),
    "enable_collect_shape": (False, "inert", _NO_PIR),
    "save_cf_stack_op": (False, "inert", _NO_PIR),
    "disable_logging_op_attr_list": ("", "inert", _NO_PIR),
    "enable_adjust_op_order": (0, "inert", _NO_PIR),
    "executor_log_deps_every_microseconds": (0, "inert", _NO_PIR),
    "cache_inference_while_scope": (False, "inert", _NO_PIR),
    "static_runtime_data_save_path": ("./", "inert", _NO_PIR),
    "save_static_runtime_data": (False, "inert", _NO_PIR),
    "tensor_operants_mode": ("eager", "inert", "one operator library serves both modes"),
    "jit_engine_type": ("Predictor", "inert", "jit.load returns a translated layer run by the same engine"),
    "enable_custom_engine": ("", "inert", _NO_PIR),
    "enable_auto_layout_pass": (False, "inert", "kernels take the layouts the layers produce"),
    "enable_fuse_parallel_matmul_pass": (True, "inert", "fusion is done in the layers (fused qkv / gate-up)"),
    "use_cinn": (False, "inert", _NO_CINN),
    "allow_cinn_ops": ("", "inert", _NO_CINN),
    "deny_cinn_ops": ("", "inert", _NO_CINN),
    "enable_cinn_compile_cache": (True, "inert", _NO_CINN),
    "cinn_compile_thread_num": (-1, "inert", _NO_CINN),
    "cinn_specify_input_dynamic_dim": (False, "inert", _NO_CINN),
    "cinn_input_dynamic_dim_spec_file": ("", "inert", _NO_CINN),
    "enable_cinn_accuracy_check": (False, "inert", _NO_CINN),
    "disable_dyshape_in_train": (False, "inert", _NO_CINN),
    "enable_fusion_fallback": (False, "inert", _NO_CINN),
    "enable_fusion_result_check": (False, "inert", _NO_CINN),
    "enable_transpose_iters_in_fusion": (True, "inert", _NO_CINN),
    "enable_reuse_iters_in_fusion": (True, "inert", _NO_CINN),
    "enable_append_iters_in_fusion": (True, "inert", _NO_CINN),
    "enable_opt_get_features": (False, "inert", _NO_PS),
    # profiler
    "host_trace_level": (1, "inert", "the activity tracer records every host category"),
    "multiple_of_cupti_buffer_size": (1, "inert", "activity buffers are sized by the tracer"),
    "trace_api": ("", "effect", "\"<file with API names>,<trace file>\" starts the API tracer"),
    # other back ends
    "use_mkldnn": (False, "inert", _NO_ONEDNN),
    "tracer_onednn_ops_on": ("", "inert", _NO_ONEDNN),
    "tracer_onednn_ops_off": ("", "inert", _NO_ONEDNN),
    "run_kp_kernel": (False, "inert", "XPU is not a target"),
    "npu_storage_format": (False, "inert", "NPU is not a target"),
    "trt_ibuilder_cache": (False, "inert", _NO_TRT),
    "trt_min_group_size": (3, "inert", _NO_TRT),
    "graph_load_in_parallel": (False, "inert", _NO_PS),
    "enable_neighbor_list_use_uva": (False, "inert", _NO_PS),
    "graph_neighbor_size_percent": (1.0, "inert", _NO_PS),
    "graph_metapath_split_opt": (False, "inert", _NO_PS),
    "graph_get_neighbor_id": (False, "inert", _NO_PS),
    "graph_embedding_split_infer_mode": (True, "inert", _NO_PS),
    "enable_graph_multi_node_sampling": (False, "inert", _NO_PS),
    "query_dest_rank_by_multi_node": (False, "inert", _NO_PS),
    "multi_node_sample_use_gpu_table": (True, "inert", _NO_PS),
    "gpugraph_storage_mode": (1, "inert", _NO_PS),
    "gpugraph_enable_hbm_table_collision_stat": (False, "inert", _NO_PS),
    "gpugraph_hbm_table_load_factor": (0.75, "inert", _NO_PS),
    "gpugraph_enable_gpu_direct_access": (False, "inert", _NO_PS),
    "gpugraph_enable_segment_merge_grads": (False, "inert", _NO_PS),
    "gpugraph_merge_grads_segment_size": (128, "inert", _NO_PS),
    "gpugraph_slot_feasign_max_num": (5, "inert", _NO_PS),
    "gpugraph_dedup_pull_push_mode": (0, "inert", _NO_PS),
    "gpugraph_load_node_list_into_hbm": (True, "inert", _NO_PS),
    "gpugraph_sparse_table_storage_mode": (0, "inert", _NO_PS),
    "gpugraph_debug_gpu_memory": (False, "inert", _NO_PS),
    # library locations
    **{f"{n}_dir": ("", "inert", _DLOPEN) for n in ("nvidia_package", "cudnn", "cuda", "cublas", "nccl", "cupti", "tensorrt", "mklml", "lapack",
                                                    "mkl", "op", "cusparselt", "curand", "cusolver", "cusparse", "win_cuda_bin")},
    # this framework's own
    "pd_wait_limit_ms": (2000, "read", "upper bound of every device-side wait in the fused communication kernels (read at import)"),
}

_flags = {}
_native_synced = False
_memory_stats_hook = False


def _parse(default, raw: str):
    if isinstance(default, bool):
        return raw.strip().lower() in ("1", "true", "yes", "on")
    if isinstance(default, int):
        return int(float(raw))
    if isinstance(default, float):
        return float(raw)
    return raw


def _coerce(name, default, value):
    """Values given to ``set_flags`` keep the flag's declared type (the reference rejects a mismatch)."""
    if isinstance(value, str) and not isinstance(default, str):
        return _parse(default, value)
    if isinstance(default, bool):
        if not isinstance(value, (bool, int)):
            raise TypeError(f"{name} expects a bool, got {type(value).__name__}")
        return bool(value)
    if isinstance(default, int):
        if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
            raise TypeError(f"{name} expects an int, got {value!r}")
        return int(value)
    if isinstance(default, float):
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise TypeError(f"{name} expects a float, got {value!r}")
        return float(value)
    return str(value)


def _init():
    for k, (default, _, _) in _SPEC.items():
        raw = os.environ.get("FLAGS_" + k)
        _flags["FLAGS_" + k] = _parse(default, raw) if raw is not None else default


_init()
# kept for readers of the earlier, flat table
_DEFAULTS = {"FLAGS_" + k: v[0] for k, v in _SPEC.items()}


def _norm(name: str) -> str:
    return name if name.startswith("FLAGS_") else "FLAGS_" + name


def _mirror_native(k, v):
    """Push one value into the native runtime's registry if that library is already loaded (never loads it)."""
    try:
        from ..ops import _lib
        rt = _lib._runtime
    except Exception:  # noqa: BLE001
        rt = None
    if rt is None:
        return False
    rt.pd_flag_set(k.encode(), (("1" if v else "0") if isinstance(v, bool) else str(v)).encode())
    return True


def sync_native():
    """Push every flag into the native runtime; called by the loader once ``libpd_runtime.so`` is open."""
    global _native_synced
    ok = False
    for k, v in _flags.items():
        ok = _mirror_native(k, v)
        if not ok:
            break
    _native_synced = ok
    return ok


def set_flags(flags: dict):
    if not isinstance(flags, dict):
        raise TypeError("flags in set_flags should be a dict")
    for k, v in flags.items():
        k = _norm(k)
        if k not in _flags:
            raise ValueError(f"Flag {k} cannot set its value through this function.")
        v = _coerce(k, _SPEC[k[6:]][0], v)
        _flags[k] = v
        _mirror_native(k, v)
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


def flag_info(name=None):
    """``{"default", "value", "kind", "note"}`` of one flag, or of all flags keyed by name."""
    if name is None:
        return {"FLAGS_" + k: flag_info(k) for k in _SPEC}
    k = _norm(name)
    if k not in _flags:
        raise ValueError(f"unknown flag {k}")
    default, kind, note = _SPEC[k[6:]]
    return {"default": default, "value": _flags[k], "kind": kind, "note": note}


def _apply_side_effect(k, v):
    import torch
    name = k[6:]
    if name == "cudnn_deterministic":
        torch.backends.cudnn.deterministic = bool(v)
    elif name == "cudnn_exhaustive_search":
        torch.backends.cudnn.benchmark = bool(v)
    elif name == "conv2d_disable_cudnn":
        torch.backends.cudnn.enabled = not bool(v)
    elif name == "enable_cublas_tensor_op_math":
        torch.backends.cuda.matmul.allow_tf32 = bool(v)
        torch.backends.cudnn.allow_tf32 = bool(v)
    elif name == "gemm_use_half_precision_compute_type":
        torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = bool(v)
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = bool(v)
    elif name == "embedding_deterministic":
        torch.use_deterministic_algorithms(bool(v), warn_only=True)
    elif name == "paddle_num_threads":
        if int(v) > 0:
            torch.set_num_threads(int(v))
    elif name == "inner_op_parallelism":
        if int(v) > 0:
            try:
                torch.set_num_interop_threads(int(v))
            except RuntimeError:
                pass                                    # parallel work already started: torch fixes the pool size then
    elif name == "check_nan_inf":
        from ..amp import debugging
        if v:
            level = int(flag("check_nan_inf_level"))
            modes = {0: debugging.DebugMode.CHECK_NAN_INF_AND_ABORT, 1: debugging.DebugMode.CHECK_NAN_INF}
            cfg = debugging.TensorCheckerConfig(enable=True, debug_mode=modes.get(level, debugging.DebugMode.CHECK_ALL)) \
                if hasattr(debugging, "TensorCheckerConfig") else None
            debugging.enable_tensor_checker(cfg)
        else:
            debugging.disable_tensor_checker()
    elif name == "low_precision_op_list":
        from ..amp import debugging
        (debugging.enable_operator_stats_collection if v else debugging.disable_operator_stats_collection)()
    elif name == "use_autotune":
        from ..ops import autotune
        autotune.set_kernel_config(enable=bool(v))
    elif name in ("fraction_of_gpu_memory_to_use", "gpu_memory_limit_mb"):
        if torch.cuda.is_available():
            if name == "gpu_memory_limit_mb":
                if int(v) > 0:
                    total = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
                    torch.cuda.set_per_process_memory_fraction(min(1.0, int(v) * 2 ** 20 / total))
            elif 0.0 < float(v) <= 1.0:
                torch.cuda.set_per_process_memory_fraction(float(v))
    elif name == "use_cuda_malloc_async_allocator":
        if v and not torch.cuda.is_initialized():
            conf = os.environ.get("PYTORCH_CUDA_ALLOC_CONF", "")
            if "backend:" not in conf:
                os.environ["PYTORCH_CUDA_ALLOC_CONF"] = (conf + "," if conf else "") + "backend:cudaMallocAsync"
    elif name in ("benchmark", "check_kernel_launch"):
        from ..ops import _lib
        _lib._sync_launches[0] = bool(flag("benchmark") or flag("check_kernel_launch"))
    elif name == "trace_api":
        from .. import api_tracer
        if v and "," in str(v):
            api_path, out_path = str(v).split(",", 1)
            api_tracer.start_api_tracer(api_path.strip(), out_path.strip())
        elif not v:
            api_tracer.stop_api_tracer()
    elif name == "log_memory_stats":
        global _memory_stats_hook
        if v and not _memory_stats_hook:
            import atexit

            def report():
                if flag("log_memory_stats") and torch.cuda.is_available() and torch.cuda.is_initialized():
                    print(torch.cuda.memory_summary(abbreviated=True))
            atexit.register(report)
            _memory_stats_hook = True
    elif name == "dataloader_use_file_descriptor":
        import torch.multiprocessing as mp
        mp.set_sharing_strategy("file_descriptor" if v else "file_system")


def _apply_env_effects():
    """Flags given through the environment act like ``set_flags`` at import (only those that differ from default)."""
    for k, (default, kind, _) in _SPEC.items():
        if kind == "effect" and _flags["FLAGS_" + k] != default:
            try:
                _apply_side_effect("FLAGS_" + k, _flags["FLAGS_" + k])
            except Exception:  # noqa: BLE001 - a flag from the environment must not break the import
                pass
