"""``DistributedStrategy`` with the reference's keys and defaults
(python/paddle/distributed/fleet/base/distributed_strategy.py; schema
paddle/fluid/framework/distributed_strategy.proto:33-134).  Nested configs are dicts with strict key
checking, as ``check_configs_key`` does."""
from __future__ import annotations

import copy

_MP_CONFIGS = {"sync_param": False, "sync_grad": False, "sync_moment": False, "sync_mode": "broadcast",
               "sync_param_name": ["embedding", "layer_norm", ".b_"], "mp_async_allreduce": False,
               "mp_skip_c_identity": False, "mp_fused_linear_param_grad_add": False, "need_broadcast_data": True,
               "recompute_allgather": False, "sp_async_reduce_scatter": False}
_PP_CONFIGS = {"dp_comm_overlap": False, "delay_scale_loss": False, "enable_timer": False,
               "sharding_comm_overlap": False, "profiling": False, "release_gradients": False,
               "overlap_p2p_comm": False, "clear_every_step_cache": False, "use_batch_p2p_comm": True,
               "best_unbalanced_scheduler": False, "micro_batch_size": 1, "accumulate_steps": 1,
               "p2p_cache_shape": True, "enable_partial_send_recv": True}
_SHARDING_CONFIGS = {"tensor_fusion": False, "accumulate_steps": 1, "comm_overlap": False, "split_param": False,
                     "fuse_optimizer": True, "use_reduce_avg": True, "comm_buffer_size_MB": 256,
                     "release_gradients": False, "enable_fuse_optimizer_states": False}
_HYBRID = {"dp_degree": -1, "mp_degree": 1, "pp_degree": 1, "sharding_degree": 1, "sep_degree": 1,
           "order": ["dp", "pp", "sharding", "sep", "mp"], "mp_configs": _MP_CONFIGS, "pp_configs": _PP_CONFIGS,
           "sharding_configs": _SHARDING_CONFIGS, "enable_optimizer_timer": False}
_AMP = {"init_loss_scaling": 32768.0, "incr_every_n_steps": 1000, "decr_every_n_nan_or_inf": 2, "incr_ratio": 2.0,
        "decr_ratio": 0.8, "use_dynamic_loss_scaling": True, "custom_white_list": [], "custom_black_list": [],
        "custom_black_varnames": [], "use_pure_fp16": False, "use_fp16_guard": True, "use_optimizer_fp16": False,
        "use_pure_bf16": False, "use_bf16_guard": False, "dtype": "float16", "level": "O1"}
_RECOMPUTE = {"checkpoints": [], "enable_offload": False, "checkpoint_shape": []}
_PIPELINE = {"micro_batch_size": 1, "accumulate_steps": 1, "schedule_mode": "1F1B", "p2p_cache_shape": True,
             "enable_partial_send_recv": True}
_TENSOR_PARALLEL = {"tensor_parallel_degree": 1, "tensor_init_seed": -1}
_GRADIENT_MERGE = {"k_steps": 1, "avg": True}
_STATIC_SHARDING = {"sharding_segment_strategy": "segment_broadcast_MB", "segment_broadcast_MB": 32.0,
                    "sharding_degree": 8, "mp_degree": 1, "dp_degree": 1, "pp_degree": 1, "stage": 1,
                    "gradient_merge_acc_step": 1, "optimize_offload": False, "hybrid_dp": False}


class _Config(dict):
    def __init__(self, name, defaults):
        super().__init__(copy.deepcopy(defaults))
        self._name = name

    def assign(self, values):
        for k, v in values.items():
            if k not in self:
                raise ValueError(f"key `{k}` is not a valid field of {self._name}")
            if isinstance(self[k], _Config) or (isinstance(self[k], dict) and isinstance(v, dict)):
                sub = self[k] if isinstance(self[k], _Config) else _Config(f"{self._name}.{k}", self[k])
                sub.assign(v)
                dict.__setitem__(self, k, sub)
            else:
                dict.__setitem__(self, k, v)

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k) from None


class DistributedStrategy:
    def __init__(self):
        d = self.__dict__
        d["_hybrid"] = _Config("hybrid_configs", _HYBRID)
        for k in ("mp_configs", "pp_configs", "sharding_configs"):
            dict.__setitem__(d["_hybrid"], k, _Config(k, _HYBRID[k]))
        d["_amp_configs"] = _Config("amp_configs", _AMP)
        d["_recompute_configs"] = _Config("recompute_configs", _RECOMPUTE)
        d["_pipeline_configs"] = _Config("pipeline_configs", _PIPELINE)
        d["_tensor_parallel_configs"] = _Config("tensor_parallel_configs", _TENSOR_PARALLEL)
        d["_gradient_merge_configs"] = _Config("gradient_merge_configs", _GRADIENT_MERGE)
        d["_sharding_configs"] = _Config("sharding_configs", _STATIC_SHARDING)
        d["_flags"] = {"amp": False, "recompute": False, "pipeline": False, "tensor_parallel": False, "sharding": False,
                       "gradient_merge": False, "lars": False, "lamb": False, "dgc": False, "localsgd": False,
                       "fuse_all_reduce_ops": True, "fuse_grad_size_in_MB": 32, "find_unused_parameters": False,
                       "without_graph_optimization": True, "heter_ccl_mode": False, "a_sync": False,
                       "sync_nccl_allreduce": True, "nccl_comm_num": 1, "fuse_grad_merge": False,
                       "fuse_grad_size_in_num": 8, "last_comm_group_size_MB": 1.0, "gradient_scale_configs":
                       {"scale_strategy": "avg"},
                       # switches of the reference's static-graph meta optimizers: kept so that strategy files load and
                       # round-trip; the dynamic-graph engine of this framework reads the hybrid / amp / recompute /
                       # sharding entries above
                       "adaptive_localsgd": False, "fp16_allreduce": False, "sync_batch_norm": False,
                       "use_hierarchical_allreduce": False, "hierarchical_allreduce_inter_nranks": 1, "asp": False,
                       "qat": False, "_calc_comm_same_stream": False, "cudnn_exhaustive_search": False,
                       "conv_workspace_size_limit": 512, "cudnn_batchnorm_spatial_persistent": False,
                       "fuse_grad_size_in_TFLOPS": 50.0, "auto": False, "semi_auto": False, "auto_search": False,
                       "split_data": True, "elastic": False,
                       "lars_configs": {"lars_coeff": 0.001, "lars_weight_decay": 0.0005, "epsilon": 0.0,
                                        "exclude_from_weight_decay": []},
                       "lamb_configs": {"lamb_weight_decay": 0.01, "exclude_from_weight_decay": []},
                       "dgc_configs": {"rampup_begin_step": 0, "rampup_step": 1, "sparsity": [0.999]},
                       "localsgd_configs": {"k_steps": 1, "begin_step": 1},
                       "adaptive_localsgd_configs": {"init_k_steps": 1, "begin_step": 1},
                       "qat_configs": {"channel_wise_abs_max": True, "weight_bits": 8, "activation_bits": 8,
                                       "not_quant_pattern": [], "algo": None}}

    hybrid_configs = property(lambda self: self._hybrid, lambda self, v: self._hybrid.assign(v))
    amp_configs = property(lambda self: self._amp_configs, lambda self, v: self._amp_configs.assign(v))
    recompute_configs = property(lambda self: self._recompute_configs, lambda self, v: self._recompute_configs.assign(v))
    pipeline_configs = property(lambda self: self._pipeline_configs, lambda self, v: self._pipeline_configs.assign(v))
    tensor_parallel_configs = property(lambda self: self._tensor_parallel_configs,
                                       lambda self, v: self._tensor_parallel_configs.assign(v))
    gradient_merge_configs = property(lambda self: self._gradient_merge_configs,
                                      lambda self, v: self._gradient_merge_configs.assign(v))
    sharding_configs = property(lambda self: self._sharding_configs, lambda self, v: self._sharding_configs.assign(v))

    def __getattr__(self, k):
        f = self.__dict__.get("_flags", {})
        if k in f:
            return f[k]
        raise AttributeError(k)

    def __setattr__(self, k, v):
        if k in self.__dict__["_flags"]:
            cur = self.__dict__["_flags"][k]
            if isinstance(cur, dict) and isinstance(v, dict) and k.endswith("_configs") and k != "gradient_scale_configs":
                unknown = set(v) - set(cur)
                if unknown:
                    raise ValueError(f"{k}: unknown keys {sorted(unknown)}")
                cur.update(v)                      # partial assignment keeps the other defaults, as in the reference
                return
            self.__dict__["_flags"][k] = v
            return
        prop = getattr(type(self), k, None)
        if isinstance(prop, property):
            prop.fset(self, v)
            return
        raise AttributeError(f"DistributedStrategy has no field {k}")

    def save_to_prototxt(self, path):
        import json
        with open(path, "w") as f:
            json.dump({"hybrid_configs": self._hybrid, "amp_configs": self._amp_configs, "flags": self._flags}, f,
                      indent=1, default=dict)

    def load_from_prototxt(self, path):
        import json
        with open(path) as f:
            d = json.load(f)
        self._hybrid.assign(d.get("hybrid_configs", {}))
        self._amp_configs.assign(d.get("amp_configs", {}))
        self._flags.update(d.get("flags", {}))

    def __repr__(self):
        return f"DistributedStrategy(hybrid_configs={dict(self._hybrid)})"
