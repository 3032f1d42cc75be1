"""``paddle.distributed.fleet.recompute.recompute_hybrid`` module path."""
from . import recompute_hybrid  # noqa: F401
