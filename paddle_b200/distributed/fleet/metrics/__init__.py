"""``paddle.distributed.fleet.metrics``: metric values reduced over all workers."""
from . import metric  # noqa: F401
from .metric import acc, auc, mae, max, min, mse, rmse, sum  # noqa: F401,A004
