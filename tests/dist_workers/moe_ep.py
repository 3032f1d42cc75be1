"""Expert parallelism over 2 ranks (2 local experts each) vs the dense evaluation of the same 4 experts on the
tokens of both ranks: outputs on this rank's tokens, gradients of this rank's experts and of its inputs
(pattern of test/collective/parallel_dygraph_moe_layer... / moe tests)."""
import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200 import nn
from paddle_b200.incubate.distributed.models.moe import MoELayer

dist.init_parallel_env()
rank, n = dist.get_rank(), dist.get_world_size()
group = dist.new_group(list(range(n)))
D, NL = 16, 2


class Expert(nn.Layer):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(D, 32)
        self.b = nn.Linear(32, D)

    def forward(self, x):
        return self.b(paddle.tanh(self.a(x)))


paddle.seed(7)
all_experts = [Expert() for _ in range(n * NL)]
local = nn.LayerList(all_experts[rank * NL:(rank + 1) * NL])
paddle.seed(8)
layer = MoELayer(D, local, gate={"type": "naive", "top_k": 2}, moe_group=group)
g = torch.Generator().manual_seed(11)
xs = [torch.randn(6 + 2 * r, D, generator=g) for r in range(n)]      # uneven token counts per rank
x = paddle.to_tensor(xs[rank].numpy()); x.stop_gradient = False
y = layer(x)
(y ** 2).sum().backward()
# dense reference on every rank's tokens
ref_grads = None
res = {}
for p in [q for e in all_experts for q in e.parameters()]:
    p._saved = p.grad.clone() if p.grad is not None else None
    p.grad = None
outs, xrefs = [], []
for r in range(n):
    xr = paddle.to_tensor(xs[r].numpy()); xr.stop_gradient = False
    val, idx = layer.gate(xr)
    out = torch.zeros_like(xr)
    rows = []
    for t in range(xr.shape[0]):
        acc = 0
        for k in range(2):
            acc = acc + val[t, k] * all_experts[int(idx[t, k])](xr[t:t + 1])[0]
        rows.append(acc)
    out = torch.stack(rows)
    (out ** 2).sum().backward()
    outs.append(out.detach()); xrefs.append(xr)
res["out"] = float((y.detach() - outs[rank]).abs().max())
res["dx"] = float((x.grad - xrefs[rank].grad).abs().max())
res["dw"] = max(float((p._saved - p.grad).abs().max()) for e in all_experts[rank * NL:(rank + 1) * NL] for p in e.parameters())
res["moe_flag"] = all(getattr(p, "is_moe_param", False) for p in local.parameters())
_common.dump(res)
