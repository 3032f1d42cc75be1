"""Tiny GPT, 10 AdamW steps under fleet (mode from argv: dp | sharding | sharding_v2 | single); dumps the
loss curve and final parameters.  The parent compares the parallel runs with the single-rank twin."""
import sys

import _common
import numpy as np
import torch

import paddle_b200 as paddle
from paddle_b200.distributed import fleet
from paddle_b200.models.gpt import GPTConfig, GPTForCausalLM

mode = sys.argv[1]
import paddle_b200.distributed as dist

if mode != "single":
    strategy = fleet.DistributedStrategy()
    n = int(__import__("os").environ["PADDLE_TRAINERS_NUM"])
    if mode == "dp":
        strategy.hybrid_configs = {"dp_degree": n}
    else:
        strategy.hybrid_configs = {"dp_degree": 1, "sharding_degree": n,
                                   "sharding_configs": {"split_param": mode == "sharding_v2"}}
    fleet.init(is_collective=True, strategy=strategy)
    rank = dist.get_rank()
else:
    n, rank = 1, 0

paddle.seed(0)
with paddle.unique_name.guard():
    model = GPTForCausalLM(GPTConfig())
opt = paddle.optimizer.AdamW(1e-3, parameters=model.parameters(), weight_decay=0.01,
                             grad_clip=paddle.nn.ClipGradByGlobalNorm(1.0))
names = [p.name for p in model.parameters()]
if mode != "single":
    model = fleet.distributed_model(model)
    opt = fleet.distributed_optimizer(opt)
world = int(sys.argv[2]) if len(sys.argv) > 2 else 2
gen = torch.Generator().manual_seed(0)
data = torch.randint(0, 1024, (10, 4 * world, 65), generator=gen)
losses = []
for step in range(10):
    batch = data[step]
    if mode != "single":
        batch = batch[rank * 4:(rank + 1) * 4]
    ids = paddle.to_tensor(batch.numpy())
    loss = model(ids[:, :-1], ids[:, 1:])
    loss.backward()
    opt.step()
    opt.clear_grad()
    losses.append(float(loss))
inner = model._layers if hasattr(model, "_layers") else model
out = {"losses": losses, "params": {k: v.numpy() for k, v in inner.state_dict().items()}, "names": names}
if rank == 0:
    import os, tempfile
    d = tempfile.mkdtemp()
    paddle.save(inner.state_dict(), os.path.join(d, "m.pdparams"))
    paddle.save(opt.state_dict(), os.path.join(d, "m.pdopt"))
    sd = paddle.load(os.path.join(d, "m.pdparams"))
    osd = paddle.load(os.path.join(d, "m.pdopt"))
    out["reload_ok"] = all(np.array_equal(sd[k].numpy(), v.numpy()) for k, v in inner.state_dict().items())
    out["opt_keys"] = sorted(k for k in osd.keys())[:6]
_common.dump(out)
