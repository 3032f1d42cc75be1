"""Plan-driven parallelisation (python/paddle/distributed/auto_parallel/intermediate/parallelize.py:49
``parallelize``; tensor_parallel.py plans ``ColWiseParallel`` :132, ``RowWiseParallel`` :226,
``SequenceParallelBegin/End/Enable/Disable`` :398-600; pipeline_parallel.py ``SplitPoint``).

``parallelize(model, optimizer, mesh, config)`` walks the sublayers, matches their names against the keys of
``config["mp_config"]["parallelize_plan"]`` (shell-style wildcards) and re-creates the matched parameters as
distributed tensors on the ``"mp"`` mesh axis; ``dp_config`` shards the inputs on the ``"dp"`` axis (and records the
sharding level); everything unmatched is replicated."""
from __future__ import annotations

import fnmatch
from enum import Enum

import torch

from ....nn.layer.layers import Layer
from ..api import ShardingStage1, ShardingStage2, ShardingStage3, shard_optimizer, shard_tensor
from ..dist_tensor import is_dist, reshard
from ..process_mesh import ProcessMesh, Replicate, Shard, get_mesh, set_mesh


class SplitPoint(Enum):
    BEGINNING = 0
    END = 1


class _Plan:
    def apply(self, layer, mesh, axis):
        raise NotImplementedError


def _set_param(layer, key, mesh, placements):
    p = layer._parameters.get(key)
    if p is not None and not is_dist(p):
        layer._parameters[key] = shard_tensor(p, mesh, placements)


def _pl(mesh, axis, p):
    out = [Replicate()] * mesh.ndim
    out[axis] = p
    return out


class ColWiseParallel(_Plan):
    """Weight split along its output columns (embedding: along the hidden size)."""

    def __init__(self, gather_output=False):
        self.gather_output = gather_output

    def apply(self, layer, mesh, axis):
        w = layer._parameters.get("weight")
        if w is None:
            return
        _set_param(layer, "weight", mesh, _pl(mesh, axis, Shard(w.dim() - 1)))
        _set_param(layer, "bias", mesh, _pl(mesh, axis, Shard(0)))
        if self.gather_output:
            layer.register_forward_post_hook(
                lambda l, i, o: reshard(o, mesh, [Replicate()] * mesh.ndim) if is_dist(o) else o)


class RowWiseParallel(_Plan):
    """Weight split along its input rows (embedding: along the vocabulary); the output is a partial sum that is
    reduced on first use."""

    def __init__(self, is_input_parallel=True):
        self.is_input_parallel = is_input_parallel

    def apply(self, layer, mesh, axis):
        _set_param(layer, "weight", mesh, _pl(mesh, axis, Shard(0)))
        _set_param(layer, "bias", mesh, [Replicate()] * mesh.ndim)


class PrepareLayerInput(_Plan):
    def __init__(self, fn=None):
        self.fn = fn

    def apply(self, layer, mesh, axis):
        if self.fn is not None:
            layer.register_forward_pre_hook(self.fn(process_mesh=mesh))


class PrepareLayerOutput(_Plan):
    def __init__(self, fn=None):
        self.fn = fn

    def apply(self, layer, mesh, axis):
        if self.fn is not None:
            layer.register_forward_post_hook(self.fn(process_mesh=mesh))


class SequenceParallelBegin(_Plan):
    """After this layer the activations are split along the sequence dimension (dim 1 of [b, s, h])."""

    def __init__(self, need_transpose=True):
        self.need_transpose = need_transpose

    def apply(self, layer, mesh, axis):
        layer.register_forward_post_hook(
            lambda l, i, o: reshard(o, mesh, _pl(mesh, axis, Shard(1))) if is_dist(o) else o)


class SequenceParallelEnd(_Plan):
    """Before this layer the sequence-split activations are gathered again."""

    def __init__(self, need_transpose=True):
        self.need_transpose = need_transpose

    def apply(self, layer, mesh, axis):
        def pre(l, inputs):
            return tuple(reshard(x, mesh, _pl(mesh, axis, Replicate())) if is_dist(x) else x for x in inputs)
        layer.register_forward_pre_hook(pre)


class SequenceParallelEnable(_Plan):
    def apply(self, layer, mesh, axis):
        def pre(l, inputs):
            return tuple(reshard(x, mesh, _pl(mesh, axis, Shard(1))) if is_dist(x) else x for x in inputs)
        layer.register_forward_pre_hook(pre)


class SequenceParallelDisable(_Plan):
    def __init__(self, need_transpose=True):
        self.need_transpose = need_transpose

    def apply(self, layer, mesh, axis):
        SequenceParallelEnd().apply(layer, mesh, axis)
        SequenceParallelBegin().apply(layer, mesh, axis)


class LocalLayer(Layer):
    """Runs ``forward`` on local shards: inputs are converted to local tensors, outputs are re-wrapped with the
    given placements (python/paddle/distributed/auto_parallel/local_layer.py)."""

    def __init__(self, out_dist_attrs, grad_dist_attrs=None):
        super().__init__()
        self.out_dist_attrs = out_dist_attrs

    def __call__(self, *inputs, **kwargs):
        from ..api import dtensor_from_local, dtensor_to_local
        inputs = [dtensor_to_local(x) if is_dist(x) else x for x in inputs]
        outs = Layer.__call__(self, *inputs, **kwargs)
        seq = list(outs) if isinstance(outs, (list, tuple)) else [outs]
        seq = [dtensor_from_local(o, m, p) for o, (m, p) in zip(seq, self.out_dist_attrs)]
        return type(outs)(seq) if isinstance(outs, (list, tuple)) else seq[0]


def parallelize(model, optimizer=None, mesh=None, config=None):
    config = config or {}
    mesh = mesh or get_mesh()
    if not isinstance(mesh, ProcessMesh):
        raise ValueError("parallelize needs a ProcessMesh (argument or paddle.distributed.auto_parallel.set_mesh)")
    set_mesh(mesh)
    names = mesh.dim_names
    if config.get("pp_config") and "pp" in names and mesh.get_dim_size("pp") > 1:
        raise NotImplementedError("pipeline splitting by plan: build the model as a fleet PipelineLayer instead")
    mp_axis = names.index("mp") if "mp" in names else None
    plan = (config.get("mp_config") or {}).get("parallelize_plan", {}) if mp_axis is not None else {}
    for name, sub in model.named_sublayers(include_self=True):
        for pattern, plans in plan.items():
            target, key = (pattern.rsplit(".", 1) + [None])[:2] if pattern.endswith((".weight", ".bias")) else (pattern, None)
            if fnmatch.fnmatch(name, target):
                for pl in (plans if isinstance(plans, (list, tuple)) else [plans]):
                    pl.apply(sub, mesh, mp_axis)
    for _, sub in model.named_sublayers(include_self=True):
        for key, p in list(sub._parameters.items()):
            if p is not None and not is_dist(p):
                sub._parameters[key] = shard_tensor(p, mesh, [Replicate()] * mesh.ndim)
    dp = config.get("dp_config") or {}
    if "dp" in names and mesh.get_dim_size("dp") > 1:
        dp_axis = names.index("dp")

        def shard_inputs(layer, inputs):
            return tuple(shard_tensor(x, mesh, _pl(mesh, dp_axis, Shard(0)))
                         if isinstance(x, torch.Tensor) and not is_dist(x) else x for x in inputs)
        model.register_forward_pre_hook(shard_inputs)
    if optimizer is not None:
        # parameters were re-created: point the optimizer at the distributed ones
        by_name = {p.name: p for p in model.parameters()}
        for g in optimizer._param_groups:
            g["params"] = [by_name.get(p.name, p) for p in g["params"]]
        optimizer._parameter_list = [p for g in optimizer._param_groups for p in g["params"]]
        level = dp.get("sharding_level", 0)
        stage = {1: ShardingStage1, 2: ShardingStage2, 3: ShardingStage3}.get(level)
        optimizer = shard_optimizer(optimizer, stage("dp", mesh) if stage else None)
    return model, optimizer


def to_distributed(model, optimizer, dataloader, device_num, node_num=1, config=None):
    """One-call helper (auto_parallel/high_level_api.py): a 1-D data-parallel mesh over ``device_num`` ranks."""
    from ..api import shard_dataloader
    mesh = ProcessMesh(list(range(device_num)), ["dp"])
    model, optimizer = parallelize(model, optimizer, mesh, {"dp_config": {"sharding_level": 0}})
    return model, optimizer, shard_dataloader(dataloader, mesh, shard_dims="dp")
