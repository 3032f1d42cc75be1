"""A plan found for a recorded model is applied to the live model on a 2-rank mesh: parameters are sharded the way the
plan says, the forward and backward run through the distributed-tensor dispatch, and outputs and gradients equal the
serial run."""
import _common
import numpy as np

import paddle_b200 as paddle
import paddle_b200.distributed as dist
import paddle_b200.nn as nn
import paddle_b200.nn.functional as F
from paddle_b200.distributed.auto_parallel import Engine
from paddle_b200.distributed.auto_parallel.static.planner import Planner
from paddle_b200.static import InputSpec

dist.init_parallel_env()
rank, n = dist.get_rank(), dist.get_world_size()


class MLP(nn.Layer):
    def __init__(self):
        super().__init__()
        self.norm, self.a, self.b = nn.LayerNorm(32), nn.Linear(32, 64), nn.Linear(64, 32)

    def forward(self, x):
        return x + self.b(F.gelu(self.a(self.norm(x))))


paddle.seed(11)
model = MLP()
x = paddle.randn([8, 32])
x.stop_gradient = False
want = model(x)
want.sum().backward()
want_grads = {k: p.grad.numpy().copy() for k, p in model.named_parameters()}
want_dx = x.grad.numpy().copy()
model.clear_gradients()

engine = Engine(model, None, None)
engine.plan([InputSpec([8, 32], "float32", "x")], n_devices=n, mode="predict")
planner = Planner(engine.main_program, n_devices=n, mesh_candidates=[(1, n)], strategies=("mp",), refine=False)
plan = planner.plan()
res = {"specs": {k: plan.dist_context.tensor_specs[s].dims_mapping for s, t in plan.dist_context.params.items()
                 for k, p in model.named_parameters() if p is t}}
mesh = plan.apply(model)
res["local_a"] = list(dist.auto_parallel.dist_tensor.local_of(model.a.weight).shape)
x2 = paddle.to_tensor(x.numpy())
x2.stop_gradient = False
xd = dist.shard_tensor(x2, mesh, [dist.Replicate(), dist.Replicate()], stop_gradient=False)
out = model(xd)
res["out_ok"] = bool(np.allclose(dist.unshard_dtensor(out).numpy(), want.numpy(), atol=1e-5))
out.sum().backward()
from paddle_b200.distributed.auto_parallel.static import Partitioner  # noqa: E402
part = Partitioner(plan.dist_context, rank)
grads = {}
for (k, p) in model.named_parameters():
    g = p.grad
    if dist.auto_parallel.is_dist(g):
        got, ref = dist.unshard_dtensor(g).numpy(), want_grads[k]
    else:                                   # the gradient of a sharded parameter is the local piece
        got = g.numpy()
        slot = [s for s, t in plan.dist_context.params.items() if list(t.shape) == list(want_grads[k].shape)
                and plan.dist_context.tensor_specs[s].dims_mapping == res["specs"][k]][0]
        ref = want_grads[k][tuple(slice(a, b) for a, b in part.local_slice(slot))]
    grads[k] = bool(got.shape == ref.shape and np.allclose(got, ref, atol=1e-4))
res["grads_ok"] = grads
_common.dump(res)
