"""Launched by ``paddle.distributed.launch``: 2-rank data-parallel training that checkpoints every step and, on the
first attempt only, loses rank 1 at step 3 (a host-side exit between steps, nothing in flight).  After the
launcher restarts the pod the run resumes from the last checkpoint; rank 0 appends ``step loss`` lines."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200 import nn

out_dir, crash = sys.argv[1], sys.argv[2] == "crash"
dist.init_parallel_env()
rank = dist.get_rank()
paddle.seed(1)
model = nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 1))
opt = paddle.optimizer.AdamW(1e-2, parameters=model.parameters())
ck_m, ck_o, ck_s = (os.path.join(out_dir, n) for n in ("m.pdparams", "m.pdopt", "step.txt"))
start = 0
if os.path.exists(ck_s):
    start = int(open(ck_s).read())
    model.set_state_dict(paddle.load(ck_m))
    opt.set_state_dict(paddle.load(ck_o))
dp = paddle.DataParallel(model)
for step in range(start, 6):
    if crash and step == 3 and rank == 1 and os.environ.get("PADDLE_RESTART_COUNT") == "0":
        sys.exit(3)
    g = torch.Generator().manual_seed(100 + step)
    x = torch.randn(8, 8, generator=g)
    y = torch.randn(8, 1, generator=g)
    sl = slice(rank * 4, rank * 4 + 4)
    loss = ((dp(paddle.to_tensor(x[sl].numpy())) - paddle.to_tensor(y[sl].numpy())) ** 2).mean()
    loss.backward()
    opt.step()
    opt.clear_grad()
    t = torch.tensor([float(loss)])
    dist.all_reduce(t)
    if rank == 0:
        paddle.save(model.state_dict(), ck_m + ".tmp"); os.replace(ck_m + ".tmp", ck_m)
        paddle.save(opt.state_dict(), ck_o + ".tmp"); os.replace(ck_o + ".tmp", ck_o)
        with open(ck_s + ".tmp", "w") as f:
            f.write(str(step + 1))
        os.replace(ck_s + ".tmp", ck_s)
        with open(os.path.join(out_dir, "loss.txt"), "a") as f:
            f.write(f"{step} {float(t) / 2:.8f}\n")
    dist.barrier()
