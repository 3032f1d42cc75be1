"""``paddle._C_ops``: operator name -> implementation registry.  The reference generates one python-C function
per entry of paddle/phi/ops/yaml/{ops,fused_ops}.yaml (python_c_gen.py:121); here each name resolves to the
implementing function of this package (hand-written kernel where one exists, torch otherwise)."""
from __future__ import annotations

import torch

from .ops import functional as _K

_REGISTRY = {}


def register(name, fn):
    _REGISTRY[name] = fn
    return fn


def _lazy(path, attr):
    def call(*a, **k):
        import importlib
        return getattr(importlib.import_module(path), attr)(*a, **k)
    return call


register("matmul", lambda x, y, transpose_x=False, transpose_y=False: _K.matmul(x, y, transpose_x, transpose_y))
register("linear", _K.linear)
register("rms_norm", lambda x, bias, residual, norm_weight, norm_bias, epsilon, begin_norm_axis, *a, **k:
         _K.rms_norm(x, norm_weight, epsilon, residual))
register("layer_norm", lambda x, scale, bias, epsilon=1e-5, begin_norm_axis=1: _K.layer_norm(x, x.shape[begin_norm_axis:], scale, bias, epsilon))
register("swiglu", _K.swiglu)
register("flash_attn", lambda q, k, v, fixed_seed_offset=None, attn_mask=None, dropout=0.0, causal=False,
         return_softmax=False, is_test=False, rng_name="": (_K.flash_attention(q, k, v, causal), None, None, None))
register("fused_rotary_position_embedding", _lazy("paddle_b200.incubate.nn.functional", "fused_rotary_position_embedding"))
register("embedding", lambda x, weight, padding_idx=-1, sparse=False: _K.embedding(x, weight, None if padding_idx < 0 else padding_idx))
register("c_embedding", lambda weight, x, start_index=0, vocab_size=-1: _K.embedding(x, weight, None, start_index, True))
register("cross_entropy_with_softmax", lambda logits, label, soft_label=False, use_softmax=True, numeric_stable_mode=True,
         ignore_index=-100, axis=-1: (torch.softmax(logits.float(), -1), _K.softmax_cross_entropy(logits, label.squeeze(-1), ignore_index).unsqueeze(-1)))
register("c_softmax_with_cross_entropy", _lazy("paddle_b200.distributed.fleet.layers.mpu.mp_ops", "_c_softmax_with_cross_entropy"))
register("c_identity", _lazy("paddle_b200.distributed.fleet.layers.mpu.mp_ops", "_c_identity"))
register("c_concat", _lazy("paddle_b200.distributed.fleet.layers.mpu.mp_ops", "_c_concat"))
register("c_split", _lazy("paddle_b200.distributed.fleet.layers.mpu.mp_ops", "_c_split"))
register("mp_allreduce_sum", _lazy("paddle_b200.distributed.fleet.layers.mpu.mp_ops", "_mp_allreduce"))
register("all_reduce", _lazy("paddle_b200.distributed.collective", "all_reduce"))
register("all_gather", _lazy("paddle_b200.distributed.collective", "all_gather"))
register("reduce_scatter", _lazy("paddle_b200.distributed.collective", "reduce_scatter"))
register("global_scatter", _lazy("paddle_b200.distributed.utils.moe_utils", "global_scatter"))
register("global_gather", _lazy("paddle_b200.distributed.utils.moe_utils", "global_gather"))
register("fused_multi_transformer_", _lazy("paddle_b200.incubate.nn.functional", "fused_multi_transformer"))
register("fused_linear_param_grad_add", _lazy("paddle_b200.incubate.nn.functional", "fused_linear_param_grad_add"))
register("skip_layernorm", _lazy("paddle_b200.incubate.nn.functional", "skip_layernorm"))
register("fused_embedding_eltwise_layernorm", _lazy("paddle_b200.incubate.nn.functional", "fused_embedding_eltwise_layernorm"))
register("fused_gate_attention", _lazy("paddle_b200.incubate.nn.functional", "fused_gate_attention"))
register("fused_dot_product_attention", _lazy("paddle_b200.incubate.nn.functional", "fused_dot_product_attention"))
register("calc_reduced_attn_scores", _lazy("paddle_b200.nn.functional.flash_attention", "calc_reduced_attention_scores"))
register("memory_efficient_attention", _lazy("paddle_b200.incubate.nn.memory_efficient_attention", "memory_efficient_attention"))
register("number_count", _lazy("paddle_b200.distributed.models.moe.utils", "_number_count"))
register("assign_pos", _lazy("paddle_b200.distributed.models.moe.utils", "_assign_pos"))
register("limit_by_capacity", _lazy("paddle_b200.distributed.models.moe.utils", "_limit_by_capacity"))
register("prune_gate_by_capacity", _lazy("paddle_b200.distributed.models.moe.utils", "_prune_gate_by_capacity"))
register("random_routing", _lazy("paddle_b200.distributed.models.moe.utils", "_random_routing"))


def __getattr__(name):
    if name in _REGISTRY:
        return _REGISTRY[name]
    import paddle_b200 as _p
    # kernel-level definitions of the later registry tiers follow the operator's own signature and output order,
    # which can differ from the same-named Python API (edit_distance, accuracy_check ...): they win
    from . import _op_table_more, _op_table_seq
    for tier in (_op_table_more, _op_table_seq):
        fn = getattr(tier, name, None)
        if callable(fn) and getattr(fn, "__module__", "") == tier.__name__ and not name.startswith("_"):
            _REGISTRY[name] = fn
            return fn
    base = name[:-1] if name.endswith("_") else name
    for mod in (_p, _p.nn.functional):
        if hasattr(mod, base):
            return getattr(mod, base)
    from . import _op_table
    fn = _op_table.resolve(name)
    if fn is not None:
        _REGISTRY[name] = fn
        return fn
    raise AttributeError(f"_C_ops has no operator {name!r}")
