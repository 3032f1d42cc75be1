"""``paddle.distributed.fleet``"""
from . import base, layers, meta_optimizers, meta_parallel, utils  # noqa: F401
from .base.distributed_strategy import DistributedStrategy  # noqa: F401
from .base.topology import CommunicateTopology, HybridCommunicateGroup, ParallelMode  # noqa: F401
from .fleet import Fleet, fleet as _fleet

init = _fleet.init
distributed_model = _fleet.distributed_model
distributed_optimizer = _fleet.distributed_optimizer
distributed_scaler = _fleet.distributed_scaler
get_hybrid_communicate_group = _fleet.get_hybrid_communicate_group
get_hybrid_parallel_topology = _fleet.get_hybrid_parallel_topology
worker_index = _fleet.worker_index
worker_num = _fleet.worker_num
node_num = _fleet.node_num
local_rank = _fleet.local_rank
is_first_worker = _fleet.is_first_worker
worker_endpoints = _fleet.worker_endpoints
barrier_worker = _fleet.barrier_worker
is_worker = _fleet.is_worker
is_server = _fleet.is_server
init_worker = _fleet.init_worker
stop_worker = _fleet.stop_worker
allreduce_perf = _fleet.allreduce_perf
broadcast_perf = _fleet.broadcast_perf
allgather_perf = _fleet.allgather_perf
reduce_scatter_perf = _fleet.reduce_scatter_perf
collective_perf = _fleet.collective_perf
fleet = _fleet
from .base.role_maker import PaddleCloudRoleMaker, Role, UserDefinedRoleMaker  # noqa: E402,F401
from .base.util_factory import UtilBase  # noqa: E402,F401
from .data_generator import MultiSlotDataGenerator, MultiSlotStringDataGenerator  # noqa: E402,F401

util = UtilBase()


def __getattr__(name):
    if name in ("recompute", "recompute_hybrid", "recompute_sequential"):
        import importlib
        r = importlib.import_module(__name__ + ".recompute")    # ("from . import" would re-enter this hook)
        return getattr(r, name) if name != "recompute" else r
    if name == "metrics":
        import importlib
        return importlib.import_module(__name__ + ".metrics")
    if name == "auto":
        from .. import auto_parallel
        return auto_parallel
    if not name.startswith("_") and hasattr(_fleet, name):
        return getattr(_fleet, name)               # every public method of the Fleet singleton is a module function
    raise AttributeError(name)
