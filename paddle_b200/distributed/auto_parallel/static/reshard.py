"""``Resharder`` under the reference's module path (python/paddle/distributed/auto_parallel/static/reshard.py)."""
from .partitioner import DistNode, Resharder, group_ranks  # noqa: F401
