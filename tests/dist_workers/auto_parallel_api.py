"""Semi-auto parallel on a 1-D mesh of 2 ranks: reshard pairs (pattern of test/auto_parallel/reshard_*.py),
SPMD matmul rules with gradients against the dense computation, data-parallel loss/gradients, and
``parallelize`` with a column/row plan against a dense twin."""
import _common
import numpy as np
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200 import nn
from paddle_b200.distributed import Partial, ProcessMesh, Replicate, Shard

dist.init_parallel_env()
rank, n = dist.get_rank(), dist.get_world_size()
mesh = ProcessMesh(list(range(n)), dim_names=["mp"])
res = {}
g = torch.Generator().manual_seed(0)
full = torch.randn(4, 6, generator=g)


def loc(t):
    return dist.auto_parallel.dtensor_to_local(t).detach().numpy()


# ---- reshard pairs
a = dist.shard_tensor(paddle.to_tensor(full.numpy()), mesh, [Shard(0)])
res["r_to_s"] = np.allclose(loc(a), full.chunk(n, 0)[rank].numpy()) and a.shape == [4, 6]
b = dist.reshard(a, mesh, [Replicate()])
res["s_to_r"] = np.allclose(loc(b), full.numpy())
c = dist.reshard(a, mesh, [Shard(1)])
res["s_to_s"] = np.allclose(loc(c), full.chunk(n, 1)[rank].numpy())
p = dist.auto_parallel.dtensor_from_local(paddle.to_tensor(full.numpy() * (rank + 1)), mesh, [Partial()])
tot = full.numpy() * sum(range(1, n + 1))
res["p_to_r"] = np.allclose(loc(dist.reshard(p, mesh, [Replicate()])), tot)
res["p_to_s"] = np.allclose(loc(dist.reshard(p, mesh, [Shard(0)])), np.split(tot, n, 0)[rank])
rp = dist.reshard(b, mesh, [Partial()])
res["r_to_p"] = np.allclose(loc(dist.reshard(rp, mesh, [Replicate()])), full.numpy())
res["unshard"] = np.allclose(dist.unshard_dtensor(c).numpy(), full.numpy())

# ---- SPMD matmul (column then row parallel) with gradients
x = torch.randn(5, 6, generator=g)
w1 = torch.randn(6, 8, generator=g, requires_grad=True)
w2 = torch.randn(8, 6, generator=g, requires_grad=True)
ref = (torch.tanh(x @ w1) @ w2).pow(2).mean()
ref.backward()
dx = dist.shard_tensor(paddle.to_tensor(x.numpy()), mesh, [Replicate()])
dw1 = dist.shard_tensor(paddle.to_tensor(w1.detach().numpy()), mesh, [Shard(1)], stop_gradient=False)
dw2 = dist.shard_tensor(paddle.to_tensor(w2.detach().numpy()), mesh, [Shard(0)], stop_gradient=False)
h = paddle.tanh(paddle.matmul(dx, dw1))
res["col_out_placement"] = repr(h.placements)
y = paddle.matmul(h, dw2)
res["row_out_placement"] = repr(y.placements)
loss = (y * y).mean()
res["mp_loss"] = abs(float(dist.unshard_dtensor(loss)) - float(ref)) < 1e-5
loss.backward()
res["mp_gw1"] = np.allclose(dw1.grad.numpy(), w1.grad.chunk(n, 1)[rank].numpy(), atol=1e-5)
res["mp_gw2"] = np.allclose(dw2.grad.numpy(), w2.grad.chunk(n, 0)[rank].numpy(), atol=1e-5)

# ---- data parallel: batch sharded, replicated weight, mean loss
xb = torch.randn(8, 6, generator=g)
w = torch.randn(6, 3, generator=g, requires_grad=True)
ref = torch.tanh(xb @ w).mean()
ref.backward()
dxb = dist.shard_tensor(paddle.to_tensor(xb.numpy()), mesh, [Shard(0)])
dw = dist.shard_tensor(paddle.to_tensor(w.detach().numpy()), mesh, [Replicate()], stop_gradient=False)
l = paddle.tanh(paddle.matmul(dxb, dw)).mean()
res["dp_loss_placement"] = repr(l.placements)
res["dp_loss"] = abs(float(dist.unshard_dtensor(l)) - float(ref)) < 1e-6
l.backward()
res["dp_gw"] = np.allclose(dw.grad.numpy(), w.grad.numpy(), atol=1e-6)


# ---- parallelize plan vs dense twin
class MLP(nn.Layer):
    def __init__(self):
        super().__init__()
        self.up = nn.Linear(6, 8)
        self.down = nn.Linear(8, 6)

    def forward(self, x):
        return self.down(paddle.tanh(self.up(x)))


paddle.seed(5)
twin, model = MLP(), MLP()
model.set_state_dict({k: v.clone() for k, v in twin.state_dict().items()})
opt_t = paddle.optimizer.AdamW(1e-2, parameters=twin.parameters())
opt = paddle.optimizer.AdamW(1e-2, parameters=model.parameters())
model, opt = dist.parallelize(model, opt, mesh, {"mp_config": {"parallelize_plan": {
    "up": dist.ColWiseParallel(), "down": dist.RowWiseParallel()}}})
res["plan_up"] = repr(model.up.weight.placements) + str(model.up.weight._local_shape)
res["plan_down"] = repr(model.down.weight.placements) + str(model.down.weight._local_shape)
lt, lp = [], []
for step in range(3):
    xin = torch.randn(4, 6, generator=g)
    a_ = (twin(paddle.to_tensor(xin.numpy())) ** 2).mean()
    a_.backward(); opt_t.step(); opt_t.clear_grad(); lt.append(float(a_))
    b_ = (model(dist.shard_tensor(paddle.to_tensor(xin.numpy()), mesh, [Replicate()])) ** 2).mean()
    b_.backward(); opt.step(); opt.clear_grad(); lp.append(float(dist.unshard_dtensor(b_)))
res["plan_losses"] = (lt, lp)
res["plan_w"] = float((dist.unshard_dtensor(model.up.weight) - twin.up.weight).abs().max())
res["opt_state_dist"] = sum(1 for v in opt.state_dict().values() if dist.auto_parallel.is_dist(v))

# ---- sharded checkpoint: save under one placement, load under another (and merged)
import os, tempfile
ck = [tempfile.mkdtemp() if rank == 0 else None]
dist.broadcast_object_list(ck, 0)
ck = ck[0]
big = torch.arange(48, dtype=torch.float32).reshape(8, 6)
sd = {"w": dist.shard_tensor(paddle.to_tensor(big.numpy()), mesh, [Shard(0)]),
      "opt": {"m": dist.shard_tensor(paddle.to_tensor(big.numpy() * 2), mesh, [Replicate()])}}
dist.save_state_dict(sd, ck)
res["ckpt_files"] = sorted(os.listdir(ck))
tgt = {"w": dist.shard_tensor(paddle.zeros([8, 6]), mesh, [Shard(1)]),
       "opt": {"m": dist.shard_tensor(paddle.zeros([8, 6]), mesh, [Shard(0)])}}
dist.load_state_dict(tgt, ck)
res["ckpt_w"] = np.allclose(loc(tgt["w"]), big.chunk(n, 1)[rank].numpy())
res["ckpt_m"] = np.allclose(loc(tgt["opt"]["m"]), (big * 2).chunk(n, 0)[rank].numpy())
from paddle_b200.distributed.checkpoint import load_merged_state_dict
merged = load_merged_state_dict(ck)
res["ckpt_merged"] = sorted(merged) == ["opt.m", "w"] and np.allclose(merged["w"].numpy(), big.numpy())
md = paddle.load(os.path.join(ck, "0.metadata"))
res["ckpt_meta"] = (type(md).__module__, sorted(md.state_dict_metadata), len(md.state_dict_metadata["w"]),
                    len(md.state_dict_metadata["opt.m"]), md.flat_mapping["opt.m"])
_common.dump(res)
