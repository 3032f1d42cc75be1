"""Rank 1 never joins the collective (it leaves between steps); rank 0's all_reduce on a group with a short
timeout must end with an error in bounded time instead of hanging."""
import datetime
import sys
import time

import _common
import torch

import paddle_b200.distributed as dist

dist.init_parallel_env()
rank = dist.get_rank()
g = dist.new_group([0, 1], timeout=datetime.timedelta(seconds=3))
x = torch.ones(4)
dist.all_reduce(x, group=g)           # one healthy collective first
if rank == 1:
    _common.dump({"left": True}, teardown=False)
    sys.exit(0)
t0 = time.time()
err = None
try:
    dist.all_reduce(x, group=g)
except Exception as e:  # noqa: BLE001
    err = type(e).__name__ + ": " + str(e)[:120]
_common.dump({"elapsed": time.time() - t0, "error": err, "first": x.tolist()}, teardown=False)
