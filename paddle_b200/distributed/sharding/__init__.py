"""``paddle.distributed.sharding`` (python/paddle/distributed/sharding/__init__.py)."""
from .group_sharded import (GroupShardedOptimizerStage2, GroupShardedScaler, GroupShardedStage2,  # noqa: F401
                            GroupShardedStage3, group_sharded_parallel, save_group_sharded_model)

__all__ = ["group_sharded_parallel", "save_group_sharded_model"]
