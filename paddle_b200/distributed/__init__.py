"""``paddle.distributed``"""
from . import collective, parallel  # noqa: F401
from .collective import (Group, P2POp, ReduceOp, all_gather, all_gather_into_tensor, all_gather_object, all_reduce,  # noqa: F401
                         all_to_all, alltoall, alltoall_single, barrier, batch_isend_irecv, broadcast,
                         broadcast_object_list, destroy_process_group, gather, gather_object, get_backend, get_group,
                         irecv, is_available, is_initialized, isend, new_group, recv, reduce, reduce_scatter, scatter,
                         scatter_object_list, send, wait)
from .parallel import DataParallel, ParallelEnv, get_rank, get_world_size, init_parallel_env  # noqa: F401

_LAZY = {"fleet", "sharding", "auto_parallel", "checkpoint", "launch", "communication", "utils", "rpc", "passes",
         "auto_tuner", "spawn_mod", "stream", "elastic", "io", "metric"}


def __getattr__(name):
    import importlib
    if name == "stream":
        return importlib.import_module(f"{__name__}.communication.stream")
    if name in _LAZY:
        try:
            return importlib.import_module(f"{__name__}.{name}")
        except ModuleNotFoundError as e:
            if e.name == f"{__name__}.{name}":
                raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
            raise
    if name == "spawn":
        from .spawn_mod import spawn
        return spawn
    if name in ("ProcessMesh", "Shard", "Replicate", "Partial", "shard_tensor", "reshard", "shard_layer",
                "shard_optimizer", "ShardingStage1", "ShardingStage2", "ShardingStage3", "dtensor_from_fn",
                "shard_dataloader", "to_static", "Strategy", "DistModel", "unshard_dtensor", "Placement",
                "parallelize", "ColWiseParallel", "RowWiseParallel", "SequenceParallelBegin", "SequenceParallelEnd",
                "SequenceParallelEnable", "SequenceParallelDisable", "SplitPoint", "PrepareLayerInput",
                "PrepareLayerOutput", "LocalLayer", "to_distributed", "DistAttr", "shard_scaler"):
        from . import auto_parallel
        return getattr(auto_parallel, name)
    if name in ("InMemoryDataset", "QueueDataset"):
        from .fleet import dataset
        return getattr(dataset, name)
    if name in ("ProbabilityEntry", "CountFilterEntry", "ShowClickEntry"):
        from . import entry_attr
        return getattr(entry_attr, name)
    if name in ("ReduceType", "set_mesh", "get_mesh"):
        from .auto_parallel import process_mesh
        return getattr(process_mesh, name)
    if name == "ParallelMode":
        from .fleet.base.topology import ParallelMode
        return ParallelMode
    if name == "split":
        from .fleet.layers.mpu.mp_ops import split
        return split
    if name in ("gloo_init_parallel_env", "gloo_barrier", "gloo_release"):
        from . import parallel
        return getattr(parallel, name)
    if name in ("save_state_dict", "load_state_dict"):
        from . import checkpoint
        return getattr(checkpoint, name)
    if name in ("group_sharded_parallel", "save_group_sharded_model"):
        from . import sharding
        return getattr(sharding, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
