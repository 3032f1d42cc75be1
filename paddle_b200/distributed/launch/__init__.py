"""``python -m paddle.distributed.launch`` (python/paddle/distributed/launch/)."""
from .main import launch  # noqa: F401
