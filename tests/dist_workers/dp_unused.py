"""DataParallel with a parameter that gets no gradient: with find_unused_parameters the pass is still finished (zeros
take part, ranks agree, the next pass starts from clean counters); without it the end of backward raises."""
import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200 import nn

dist.init_parallel_env()
rank = dist.get_rank()


class Net(nn.Layer):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(4, 4)
        self.unused = nn.Linear(4, 4)

    def forward(self, x, use_all=False):
        y = self.a(x)
        return y + self.unused(x) if use_all else y


paddle.seed(1)
res = {}
net = paddle.DataParallel(Net(), find_unused_parameters=True)
x = paddle.to_tensor(torch.full((2, 4), float(rank + 1)).numpy())
for step in range(2):                       # two passes: stale counters from the first would corrupt the second
    net(x).sum().backward()
g = net._layers.a.weight.grad
t = g.clone(); dist.all_reduce(t)
res["agree"] = bool(torch.allclose(t / 2, g))
res["unused_zero"] = bool(net._layers.unused.weight.grad is not None and float(net._layers.unused.weight.grad.abs().sum()) == 0.0)
res["expected"] = bool(torch.allclose(g[0], torch.full((4,), 2 * 2 * 1.5)))   # 2 passes x 2 rows x mean(1, 2)
strict = paddle.DataParallel(Net(), find_unused_parameters=False)
try:
    strict(x).sum().backward()
    res["raised"] = False
except RuntimeError as e:
    res["raised"] = "find_unused_parameters" in str(e)
# the collective sequence stays aligned afterwards
strict(x, use_all=True).sum().backward()
res["after_ok"] = strict._layers.unused.weight.grad is not None
_common.dump(res)
