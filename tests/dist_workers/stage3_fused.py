"""group_sharded_parallel(level="p_g_os") on GPUs with bf16 Linear layers: the layers run on the fused gather->GEMM /
GEMM->reduce-scatter kernels (no full weight in training); losses and final weights follow a single-process twin
that sees the whole batch."""
import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200 import nn
from paddle_b200.distributed.sharding import group_sharded_parallel
from paddle_b200.ops import _lib, native

dist.init_parallel_env()
rank, n = dist.get_rank(), dist.get_world_size()


class MLP(nn.Layer):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(256, 512)
        self.fc2 = nn.Linear(512, 256)
        self.head = nn.Linear(256, 128)          # in / n = 128 rows per slice: fused as well

    def forward(self, x):
        return self.head(paddle.tanh(self.fc2(paddle.tanh(self.fc1(x)))))


paddle.seed(3)
twin = MLP().to("gpu").to(dtype="bfloat16")
model = MLP().to("gpu").to(dtype="bfloat16")
model.set_state_dict({k: v.clone() for k, v in twin.state_dict().items()})
opt_t = paddle.optimizer.AdamW(1e-3, parameters=twin.parameters(), multi_precision=True)
opt = paddle.optimizer.AdamW(1e-3, parameters=model.parameters(), multi_precision=True)
wrapped, opt, _ = group_sharded_parallel(model, opt, "p_g_os")
fused_units = sum(1 for u in wrapped._units if getattr(u, "fused_weight", None) is not None)
gen = torch.Generator().manual_seed(1)
lt, lp = [], []
l0 = native.LAUNCH_COUNT
for step in range(4):
    xb = torch.randn(128 * n, 256, generator=gen).bfloat16().cuda()
    yb = torch.randint(0, 100, (128 * n,), generator=gen).cuda()
    a = paddle.nn.functional.cross_entropy(twin(paddle.to_tensor(xb)).astype("float32"), paddle.to_tensor(yb))
    a.backward(); opt_t.step(); opt_t.clear_grad(); lt.append(float(a))
    sl = slice(rank * 128, rank * 128 + 128)
    b = paddle.nn.functional.cross_entropy(wrapped(paddle.to_tensor(xb[sl])).astype("float32"), paddle.to_tensor(yb[sl]))
    b.backward(); opt.step(); opt.clear_grad()
    t = torch.tensor([float(b)], device="cuda"); dist.all_reduce(t); lp.append(float(t) / n)
torch.cuda.synchronize()
_lib.check_status()
sd = wrapped.state_dict()
maxdiff = max(float((sd[k].float() - v.float()).abs().max()) for k, v in twin.state_dict().items())
_common.dump({"twin": lt, "sharded": lp, "maxdiff": maxdiff, "fused_units": fused_units,
              "launches": native.LAUNCH_COUNT - l0})
