"""``paddle.incubate.distributed.fleet``: recompute entry points for hybrid-parallel and sequential models."""
from ....distributed.fleet.recompute import recompute_hybrid, recompute_sequential  # noqa: F401

__all__ = ["recompute_sequential", "recompute_hybrid"]
