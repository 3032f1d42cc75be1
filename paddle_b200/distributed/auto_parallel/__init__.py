"""``paddle.distributed.auto_parallel``: process meshes, placements, distributed tensors, reshard."""
from .api import (DistModel, ShardDataloader, ShardingStage1, ShardingStage2, ShardingStage3, Strategy,  # noqa: F401
                  dtensor_from_fn, dtensor_from_local, dtensor_to_local, shard_dataloader, shard_layer,
                  shard_optimizer, shard_scaler, shard_tensor, to_static, unshard_dtensor, moe_global_mesh_tensor,
                  moe_sub_mesh_tensors, in_auto_parallel_align_mode, FusePasses)
from .dist_tensor import DistTensor, is_dist, reshard  # noqa: F401
from .intermediate import (ColWiseParallel, LocalLayer, PrepareLayerInput, PrepareLayerOutput, RowWiseParallel,  # noqa: F401
                           SequenceParallelBegin, SequenceParallelDisable, SequenceParallelEnable,
                           SequenceParallelEnd, SplitPoint, parallelize, to_distributed)
from .process_mesh import (Partial, Placement, ProcessMesh, ReduceType, Replicate, Shard, get_mesh,  # noqa: F401
                           set_mesh)

DistAttr = dict
from .engine import Engine  # noqa: F401,E402
