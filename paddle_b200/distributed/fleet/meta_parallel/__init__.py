"""Model wrappers applied by ``fleet.distributed_model`` (python/paddle/distributed/fleet/meta_parallel/):
they broadcast the replicated parameters inside the relevant groups at wrap time
(fleet/utils/hybrid_parallel_util.py:225-246) and forward everything else to the wrapped layer."""
from __future__ import annotations

import torch

from ....nn.layer.layers import Layer
from ... import collective as C
from ..utils.hybrid_parallel_util import (broadcast_dp_parameters, broadcast_mp_parameters,
                                          broadcast_sep_parameters, broadcast_sharding_parameters)


class MetaParallelBase(Layer):
    def __init__(self, layers, hcg, strategy=None):
        super().__init__()
        self._layers = layers
        self._hcg = hcg
        self._strategy = strategy
        self._prepare_for_model()

    def _prepare_for_model(self):
        pass

    def forward(self, *inputs, **kwargs):
        return self._layers(*inputs, **kwargs)

    def state_dict(self, *a, **k):
        return self._layers.state_dict(*a, **k)

    def set_state_dict(self, *a, **k):
        return self._layers.set_state_dict(*a, **k)

    set_dict = load_dict = set_state_dict

    def parameters(self, include_sublayers=True):
        return self._layers.parameters(include_sublayers)

    def named_parameters(self, prefix="", include_sublayers=True):
        return self._layers.named_parameters(prefix, include_sublayers)


class TensorParallel(MetaParallelBase):
    def _prepare_for_model(self):
        broadcast_mp_parameters(self._layers, self._hcg)
        if self._hcg.get_sharding_parallel_world_size() > 1:
            broadcast_sharding_parameters(self._layers, self._hcg)
        if self._hcg.get_data_parallel_world_size() > 1:
            broadcast_dp_parameters(self._layers, self._hcg)


class ShardingParallel(MetaParallelBase):
    def _prepare_for_model(self):
        broadcast_sharding_parameters(self._layers, self._hcg)
        if self._hcg.get_data_parallel_world_size() > 1:
            broadcast_dp_parameters(self._layers, self._hcg)


class SegmentParallel(MetaParallelBase):
    def _prepare_for_model(self):
        broadcast_sep_parameters(self._layers, self._hcg)
        if self._hcg.get_sharding_parallel_world_size() > 1:
            broadcast_sharding_parameters(self._layers, self._hcg)
        if self._hcg.get_data_parallel_world_size() > 1:
            broadcast_dp_parameters(self._layers, self._hcg)


def __getattr__(name):
    if name in ("PipelineParallel", "PipelineParallelWithInterleave", "PipelineParallelWithInterleaveFthenB",
                "PipelineParallelWithInterleaveWindowed"):
        from . import pipeline_parallel as pp
        return getattr(pp, name)
    if name in ("RNGStatesTracker", "get_rng_state_tracker", "model_parallel_random_seed"):
        from ..layers.mpu import random as _r
        return getattr(_r, name)
    if name in ("LayerDesc", "SharedLayerDesc", "PipelineLayer", "SegmentLayers"):
        from .parallel_layers import pp_layers
        return getattr(pp_layers, name)
    if name in ("VocabParallelEmbedding", "ColumnParallelLinear", "RowParallelLinear", "ParallelCrossEntropy"):
        from ..layers.mpu import mp_layers
        return getattr(mp_layers, name)
    if name in ("get_rng_state_tracker", "model_parallel_random_seed"):
        from ..layers.mpu import random as r
        return getattr(r, name)
    raise AttributeError(name)
