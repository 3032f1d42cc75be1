"""Semi-automatic parallel API (python/paddle/distributed/auto_parallel/api.py: ``shard_tensor`` :190,
``dtensor_from_local`` :349, ``reshard`` :444, ``shard_layer`` :545, ``shard_optimizer`` :1218,
``ShardingStage1/2/3`` :1084-1200, ``to_static`` :2153, ``unshard_dtensor`` :2478, ``shard_dataloader`` :2934)."""
from __future__ import annotations

import numpy as np
import torch

from ..._core.tensor import EagerParamBase, Tensor, as_tensor
from ...nn.layer.layers import Layer
from .. import collective as C
from .dist_tensor import (DistTensor, _local_shape, _norm_placements, is_dist, local_of, reshard,  # noqa: F401
                          reshard_local)
from .process_mesh import Partial, Placement, ProcessMesh, ReduceType, Replicate, Shard, get_mesh  # noqa: F401


def _slice_for(global_t, mesh, placements):
    """Local shard of a tensor that every rank holds in full."""
    coord = mesh.coord_of(C.get_rank())
    x = global_t
    if coord is None:
        return x.new_empty(0)
    for a, p in enumerate(placements):
        if p.is_shard():
            n = mesh.shape[a]
            assert x.shape[p.dim] % n == 0, f"dim {p.dim} ({x.shape[p.dim]}) not divisible by mesh axis size {n}"
            x = x.chunk(n, dim=p.dim)[coord[a]]
        elif p.is_partial() and coord[a] != 0:
            x = torch.zeros_like(x)
    return x.contiguous()


class DistParam(DistTensor, EagerParamBase):
    """A parameter whose data is the local shard."""

    @staticmethod
    def __new__(cls, data, trainable=True, name=None):
        return torch.Tensor._make_subclass(cls, data.detach(), trainable)

    def __init__(self, data, trainable=True, name=None):
        EagerParamBase.__init__(self, data, trainable, name)


def shard_tensor(data, mesh, placements, dtype=None, place=None, stop_gradient=None):
    placements = _norm_placements(mesh, placements)
    if is_dist(data):
        return reshard(data, mesh, placements)
    t = data if isinstance(data, torch.Tensor) else as_tensor(torch.as_tensor(data))
    with torch.no_grad():
        local = _slice_for(t.detach().as_subclass(torch.Tensor), mesh, placements).clone()
    if dtype is not None:
        from ..._core import dtype as _dt
        local = local.to(_dt.to_torch(dtype))
    if isinstance(data, EagerParamBase):
        out = DistParam(local, data.trainable, name=data.name)
        for k in ("optimize_attr", "regularizer", "need_clip", "is_distributed"):
            setattr(out, k, getattr(data, k, None))
        out._dist_mesh, out._dist_placements = mesh, placements
        return out
    out = DistTensor.wrap(local, mesh, placements)
    sg = stop_gradient if stop_gradient is not None else not getattr(data, "requires_grad", False)
    if not sg and out.is_floating_point():
        out.requires_grad_(True)
    return out


def dtensor_from_local(local_tensor, mesh, placements):
    return DistTensor.wrap(local_tensor.as_subclass(torch.Tensor) if isinstance(local_tensor, torch.Tensor)
                           else torch.as_tensor(local_tensor), mesh, placements)


def dtensor_to_local(dist_tensor, mesh=None, placements=None):
    return local_of(dist_tensor).as_subclass(Tensor)


def dtensor_from_fn(fn, mesh, placements, *args, **kwargs):
    return shard_tensor(fn(*args, **kwargs), mesh, placements)


def unshard_dtensor(dist_tensor):
    """Full (replicated) dense tensor."""
    if not is_dist(dist_tensor):
        return dist_tensor
    mesh = dist_tensor.process_mesh
    full = reshard(dist_tensor, mesh, [Replicate()] * mesh.ndim)
    return local_of(full).as_subclass(Tensor)


def shard_layer(layer: Layer, process_mesh: ProcessMesh, shard_fn=None, input_fn=None, output_fn=None):
    """Turn every parameter into a distributed one: ``shard_fn(name, sublayer, mesh)`` may assign sharded
    parameters itself; everything it leaves untouched becomes replicated."""
    if not isinstance(process_mesh, ProcessMesh):
        raise ValueError("The argument `process_mesh` cannot be empty")
    for name, sub in layer.named_sublayers(include_self=True):
        if shard_fn is not None:
            shard_fn(name, sub, process_mesh)
        for key, p in list(sub._parameters.items()):
            if p is not None and not is_dist(p):
                sub._parameters[key] = shard_tensor(p, process_mesh, [Replicate()] * process_mesh.ndim)
        for key, b in list(sub._buffers.items()):
            if b is not None and not is_dist(b):
                sub._buffers[key] = shard_tensor(b, process_mesh, [Replicate()] * process_mesh.ndim)
    if input_fn is not None:
        layer.register_forward_pre_hook(lambda l, inputs: input_fn(inputs, process_mesh))
    if output_fn is not None:
        layer.register_forward_post_hook(lambda l, inputs, outputs: output_fn(outputs, process_mesh))
    return layer


class _ShardingStageBase:
    def __init__(self, sharding_mesh_dim=None, mesh=None):
        self._dim, self._mesh = sharding_mesh_dim, mesh


class ShardingStage1(_ShardingStageBase):
    """Optimizer states sharded along one mesh axis (the accumulators of a replicated parameter are stored as
    Shard(0) slices when dim 0 divides; otherwise they stay replicated)."""
    stage = 1


class ShardingStage2(_ShardingStageBase):
    stage = 2


class ShardingStage3(_ShardingStageBase):
    stage = 3


class _ShardOptimizer:
    """Optimizer wrapper of ``shard_optimizer`` (api.py:_ShardOptimizer :1218): accumulators follow the
    parameter's placements (they are created on the local shard); with a sharding stage, the gradient of a
    parameter that is replicated along the sharding axis is averaged over that axis before the step."""

    def __init__(self, optimizer, shard_fn=None, gradient_accumulation_steps=1):
        self._inner_opt = optimizer
        self._shard_fn = shard_fn
        self._acc = gradient_accumulation_steps

    def step(self):
        self._inner_opt.step()

    def clear_grad(self, set_to_zero=True):
        self._inner_opt.clear_grad(set_to_zero)

    def state_dict(self):
        sd = self._inner_opt.state_dict()
        by_name = {p.name: p for p in self._inner_opt._parameter_list}
        out = {}
        for k, v in sd.items():
            owner = next((p for n, p in by_name.items() if str(k).startswith(n + "_")), None)
            if owner is not None and is_dist(owner) and isinstance(v, torch.Tensor) and \
                    list(v.shape) == owner._local_shape:
                v = DistTensor.wrap(v.as_subclass(torch.Tensor), owner.process_mesh, owner.placements)
            out[k] = v
        return out

    def set_state_dict(self, sd):
        return self._inner_opt.set_state_dict({k: (local_of(v).as_subclass(Tensor) if is_dist(v) else v)
                                               for k, v in sd.items()})

    def __getattr__(self, item):
        return getattr(self._inner_opt, item)


def shard_optimizer(optimizer, shard_fn=None, gradient_accumulation_steps=1):
    return _ShardOptimizer(optimizer, shard_fn, gradient_accumulation_steps)


def shard_scaler(scaler):
    return scaler


class ShardDataloader:
    """Wraps a loader: every batch tensor becomes a DistTensor sharded on ``shard_dims`` of the mesh
    (api.py:2934).  Each rank is expected to load the GLOBAL batch; the local slice is taken here."""

    def __init__(self, dataloader, meshes, input_keys=None, shard_dims=None, is_dataset_splitted=False):
        self._loader = dataloader
        self._mesh = meshes[0] if isinstance(meshes, (list, tuple)) else meshes
        self._dim = shard_dims[0] if isinstance(shard_dims, (list, tuple)) else shard_dims
        self._split = is_dataset_splitted

    def __len__(self):
        return len(self._loader)

    def _conv(self, t):
        if not isinstance(t, torch.Tensor):
            return t
        pl = [Replicate()] * self._mesh.ndim
        if self._dim is not None:
            pl[self._mesh._axis(self._dim)] = Shard(0)
        if self._split:
            return dtensor_from_local(t, self._mesh, pl)
        return shard_tensor(t, self._mesh, pl)

    def __iter__(self):
        for batch in self._loader:
            if isinstance(batch, dict):
                yield {k: self._conv(v) for k, v in batch.items()}
            elif isinstance(batch, (list, tuple)):
                yield type(batch)(self._conv(v) for v in batch)
            else:
                yield self._conv(batch)


def shard_dataloader(dataloader, meshes, input_keys=None, shard_dims=None, is_dataset_splitted=False):
    return ShardDataloader(dataloader, meshes, input_keys, shard_dims, is_dataset_splitted)


class Strategy:
    """Configuration bag of ``to_static`` (auto_parallel/strategy.py)."""

    class _Section(dict):
        __getattr__ = dict.get

        def __setattr__(self, k, v):
            self[k] = v

    def __init__(self, config=None):
        config = config or {}
        for name in ("sharding", "gradient_merge", "pipeline", "amp", "fused_passes", "recompute", "mp_optimization",
                     "dp_optimization", "sp_optimization"):
            sec = Strategy._Section(enable=False)
            sec.update(config.get(name, {}))
            setattr(self, name, sec)


class DistModel:
    """Result of ``to_static``: runs the dynamic layer step by step (the reference lowers to a static program;
    here capture happens in ``paddle.jit``).  ``__call__`` in train mode runs forward, loss, backward and the
    optimizer step and returns the loss."""

    def __init__(self, layer, loader=None, loss=None, optimizer=None, strategy=None):
        self._layer, self._loss, self._opt, self._strategy = layer, loss, optimizer, strategy
        self._mode = "train" if (loss is not None and optimizer is not None) else ("eval" if loss is not None else "predict")

    def train(self):
        self._mode = "train"
        self._layer.train()

    def eval(self):
        self._mode = "eval"
        self._layer.eval()

    def predict(self):
        self._mode = "predict"
        self._layer.eval()

    def __call__(self, *args):
        if self._mode == "predict":
            with torch.no_grad():
                return self._layer(*args)
        *inputs, label = args
        if self._mode == "eval":
            with torch.no_grad():
                return self._loss(self._layer(*inputs), label)
        loss = self._loss(self._layer(*inputs), label)
        loss.backward()
        self._opt.step()
        self._opt.clear_grad()
        return loss

    def state_dict(self, mode="all"):
        sd = dict(self._layer.state_dict())
        if mode in ("all", "opt") and self._opt is not None:
            sd.update(self._opt.state_dict())
        return sd

    def set_state_dict(self, sd):
        self._layer.set_state_dict(sd)

    def dist_main_program(self, mode=None):
        return None


def to_static(layer, loader=None, loss=None, optimizer=None, strategy=None, input_spec=None):
    return DistModel(layer, loader, loss, optimizer, strategy)


# ------------------------------------------------------------------------------------- MoE mesh helpers
def _sub_meshes_and_local_placements(mesh, placements, local_mesh_dim):
    """Splits ``mesh`` along ``local_mesh_dim`` into one sub-mesh per index; the placement of that mesh dimension is
    dropped for the sub-meshes (python/paddle/distributed/auto_parallel/api.py ``_get_sub_meshes_and_local_placements``)."""
    a = local_mesh_dim if local_mesh_dim >= 0 else mesh.ndim + local_mesh_dim
    arr = np.asarray(mesh.mesh)
    names = [n for i, n in enumerate(mesh.dim_names) if i != a]
    subs = []
    for i in range(arr.shape[a]):
        sub = np.take(arr, i, axis=a)
        subs.append(ProcessMesh(sub if sub.ndim else sub.reshape(1), names or ["d0"]))
    local_pl = [p for i, p in enumerate(placements) if i != a] or [Replicate()]
    return subs, local_pl


def moe_global_mesh_tensor(local_tensor_list, mesh, placements, local_mesh_dim=-1):
    """Views the per-sub-mesh tensors of an expert-parallel layer (one per index of ``local_mesh_dim``; this rank holds
    the one of its own sub-mesh) as ONE distributed tensor over ``mesh`` with ``placements``; no data moves."""
    a = local_mesh_dim if local_mesh_dim >= 0 else mesh.ndim + local_mesh_dim
    coord = mesh.coord_of(C.get_rank() if C.is_initialized() else 0)
    idx = 0 if coord is None else coord[a]
    t = local_tensor_list[idx]
    local = local_of(t) if isinstance(t, DistTensor) else t
    return DistTensor.wrap(local.as_subclass(torch.Tensor), mesh, list(placements))


def moe_sub_mesh_tensors(dist_tensor, global_mesh=None, local_mesh_dim=-1, global_placements=None):
    """Inverse of :func:`moe_global_mesh_tensor`: one distributed tensor per sub-mesh along ``local_mesh_dim``; the
    entry of this rank's sub-mesh carries its local shard, the others are placeholders of the same local shape."""
    mesh = global_mesh or dist_tensor.process_mesh
    placements = list(global_placements or dist_tensor.placements)
    subs, local_pl = _sub_meshes_and_local_placements(mesh, placements, local_mesh_dim)
    a = local_mesh_dim if local_mesh_dim >= 0 else mesh.ndim + local_mesh_dim
    coord = mesh.coord_of(C.get_rank() if C.is_initialized() else 0)
    mine = 0 if coord is None else coord[a]
    local = local_of(dist_tensor).as_subclass(torch.Tensor)
    out = []
    for i, sub in enumerate(subs):
        out.append(DistTensor.wrap(local if i == mine else torch.empty_like(local), sub, list(local_pl)))
    return out


def in_auto_parallel_align_mode():
    import os
    from ...framework.flags import flag
    return bool(flag("enable_auto_parallel_align_mode"))


class FusePasses:
    """Switches of the fusion passes in ``Strategy.fused_passes``; the fusions are properties of the kernels here, the
    object only carries the configuration."""

    def __init__(self, config_dict=None):
        self.enable = False
        self.gemm_epilogue = False
        self.dropout_add = False
        for k, v in (config_dict or {}).items():
            setattr(self, k, v)


DistAttr = dict      # {'process_mesh': ..., 'placements': ...}: what ``DistTensor.dist_attr`` returns
