"""group_sharded_parallel (levels os / os_g / p_g_os) vs a single-process twin trained on the whole batch
(pattern of test/collective/fleet/dygraph_group_sharded_stage2.py / _stage3.py)."""
import os
import sys
import tempfile

import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200 import nn
from paddle_b200.distributed.sharding import group_sharded_parallel, save_group_sharded_model

level = sys.argv[1]
dist.init_parallel_env()
rank, n = dist.get_rank(), dist.get_world_size()


class MLP(nn.Layer):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(50, 24)
        self.fc1 = nn.Linear(24, 40)
        self.norm = nn.LayerNorm(40)
        self.fc2 = nn.Linear(40, 50)

    def forward(self, ids):
        return self.fc2(self.norm(paddle.tanh(self.fc1(self.emb(ids)))))


paddle.seed(3)
twin = MLP()
model = MLP()
model.set_state_dict({k: v.clone() for k, v in twin.state_dict().items()})
clip = paddle.nn.ClipGradByGlobalNorm(0.5)
opt_t = paddle.optimizer.AdamW(1e-2, parameters=twin.parameters(), grad_clip=clip)
opt = paddle.optimizer.AdamW(1e-2, parameters=model.parameters(), grad_clip=paddle.nn.ClipGradByGlobalNorm(0.5))
wrapped, opt, _ = group_sharded_parallel(model, opt, level)
gen = torch.Generator().manual_seed(1)
lt, lp = [], []
for step in range(4):
    ids = torch.randint(0, 50, (4 * n, 6), generator=gen)
    lab = torch.randint(0, 50, (4 * n, 6), generator=gen)
    a = paddle.nn.functional.cross_entropy(twin(paddle.to_tensor(ids.numpy())).reshape([-1, 50]),
                                           paddle.to_tensor(lab.numpy()).reshape([-1]))
    a.backward(); opt_t.step(); opt_t.clear_grad(); lt.append(float(a))
    sl = slice(rank * 4, rank * 4 + 4)
    b = paddle.nn.functional.cross_entropy(wrapped(paddle.to_tensor(ids[sl].numpy())).reshape([-1, 50]),
                                           paddle.to_tensor(lab[sl].numpy()).reshape([-1]))
    b.backward(); opt.step(); opt.clear_grad()
    t = torch.tensor([float(b)]); dist.all_reduce(t); lp.append(float(t) / n)

# ---- loss scaling through the scaler that group_sharded_parallel returns: a step whose loss is inf on rank 1 only must
# be skipped on BOTH ranks; the next (finite) scaled step must equal the twin's plain step
scaler_res = None
if len(sys.argv) > 2 and sys.argv[2] == "scaler":
    from paddle_b200.amp import GradScaler
    from paddle_b200.distributed.sharding.group_sharded import GroupShardedScaler
    scaler = GroupShardedScaler(GradScaler(init_loss_scaling=1024.0, decr_every_n_nan_or_inf=1))
    before = {k: v.clone() for k, v in wrapped.state_dict().items()}
    ids = torch.randint(0, 50, (4, 6), generator=gen)
    out = wrapped(paddle.to_tensor(ids.numpy())).sum()
    bad = out * (float("inf") if rank == 1 else 1.0)
    scaler.scale(bad).backward()
    scaler.step(opt); scaler.update(); opt.clear_grad()
    after = wrapped.state_dict()
    skipped = max(float((after[k].float() - v.float()).abs().max()) for k, v in before.items())
    scale_after_inf = scaler._scale
    ids = torch.randint(0, 50, (4 * n, 6), generator=gen)
    lab = torch.randint(0, 50, (4 * n, 6), generator=gen)
    a = paddle.nn.functional.cross_entropy(twin(paddle.to_tensor(ids.numpy())).reshape([-1, 50]),
                                           paddle.to_tensor(lab.numpy()).reshape([-1]))
    a.backward(); opt_t.step(); opt_t.clear_grad()
    sl = slice(rank * 4, rank * 4 + 4)
    b = paddle.nn.functional.cross_entropy(wrapped(paddle.to_tensor(ids[sl].numpy())).reshape([-1, 50]),
                                           paddle.to_tensor(lab[sl].numpy()).reshape([-1]))
    scaler.scale(b).backward(); scaler.step(opt); scaler.update(); opt.clear_grad()
    scaler_res = {"skipped_maxdiff": skipped, "scale_after_inf": scale_after_inf}

sd = wrapped.state_dict()
maxdiff = max(float((sd[k].float() - v.float()).abs().max()) for k, v in twin.state_dict().items())
nstate = len(opt.state_dict())
out = tempfile.mkdtemp()
save_group_sharded_model(wrapped, out, opt)
files = sorted(os.listdir(out))
_common.dump({"scaler": scaler_res, "twin": lt, "sharded": lp, "maxdiff": maxdiff, "nstate": nstate, "files": files})
