"""``paddle.distributed.fleet.recompute.recompute`` module path (python/paddle/distributed/fleet/recompute/recompute.py)."""
from . import RecomputeFunction, recompute, recompute_sequential  # noqa: F401
