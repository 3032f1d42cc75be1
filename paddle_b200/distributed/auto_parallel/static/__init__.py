"""Planner for recorded programs (python/paddle/distributed/auto_parallel/static/): cluster description, completion of
sharding annotations through the SPMD rules, operator and communication cost model, rule-based search for a data /
tensor parallel plan, and the per-rank partition of a completed program."""
from .cluster import Cluster, Device, DeviceType, Link, LinkType, Machine, get_default_cluster  # noqa: F401
from .completion import CommStep, Completer, DistContext, DistOp, Reshard  # noqa: F401
from .cost import CommContext, Cost, CostEstimator  # noqa: F401
from .partitioner import DistNode, Partitioner, Resharder, group_ranks  # noqa: F401
from .planner import ParallelTuner, Plan, Planner, RuleBasedTuner  # noqa: F401
