"""Fused all-gather->GEMM and GEMM->reduce-scatter vs NCCL + fp32 reference, fwd and bwd, several calls in
a row (exercises the epoch / ack protocol), plus timings against the unfused NCCL + cuBLAS sequence."""
import os
import sys

import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200.distributed import fleet
from paddle_b200.ops import _lib

n = int(os.environ["PADDLE_TRAINERS_NUM"])
strategy = fleet.DistributedStrategy()
strategy.hybrid_configs = {"dp_degree": 1, "mp_degree": n}
fleet.init(is_collective=True, strategy=strategy)
rank = dist.get_rank()
g = fleet.get_hybrid_communicate_group().get_model_parallel_group()
from paddle_b200.parallel import fused_linear_impl as FL
from paddle_b200.distributed.fleet.utils import sequence_parallel_utils as spu

big = len(sys.argv) > 1 and sys.argv[1] == "big"
T, H, F = (4096, 4096, 11008 // n // 8 * 8 * 2) if big else (1024, 512, 768)
rows = T // n
torch.manual_seed(100 + rank)
res = {"errs": {}}


def rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))


for it in range(3):
    x = (torch.randn(rows, H, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(H, F, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    # ---- all-gather -> GEMM, forward + backward
    y = FL.allgather_linear(x, w, g)
    dy = (torch.randn(T, F, device="cuda") * 0.1).to(torch.bfloat16)
    y.backward(dy)
    xf = spu.all_gather(x.detach(), g).float()
    ref_y = xf @ w.detach().float()
    ref_dx_full = dy.float() @ w.detach().float().t()
    dist.all_reduce(ref_dx_full, group=g)
    ref_dx = ref_dx_full[rank * rows:(rank + 1) * rows]
    ref_dw = xf.t() @ dy.float()
    res["errs"][f"ag_y_{it}"] = rel(y, ref_y)
    res["errs"][f"ag_dx_{it}"] = rel(x.grad, ref_dx)
    res["errs"][f"ag_dw_{it}"] = rel(w.grad, ref_dw)
    # ---- GEMM -> reduce-scatter, forward + backward
    x2 = (torch.randn(T, F, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w2 = (torch.randn(F, H, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    y2 = FL.linear_reduce_scatter(x2, w2, g)
    dy2 = (torch.randn(rows, H, device="cuda") * 0.1).to(torch.bfloat16)
    y2.backward(dy2)
    full = x2.detach().float() @ w2.detach().float()
    dist.all_reduce(full, group=g)
    ref_y2 = full[rank * rows:(rank + 1) * rows]
    dyf = spu.all_gather(dy2, g).float()
    res["errs"][f"rs_y_{it}"] = rel(y2, ref_y2)
    res["errs"][f"rs_dx_{it}"] = rel(x2.grad, dyf @ w2.detach().float().t())
    res["errs"][f"rs_dw_{it}"] = rel(w2.grad, x2.detach().float().t() @ dyf)
# ---- row-parallel layer without sequence parallelism: GEMM -> reduce-scatter kernel + gather = all-reduce, through the
# public layer (RowParallelLinear with input_is_parallel), forward and backward against fp32
from paddle_b200.distributed.fleet.layers.mpu.mp_layers import RowParallelLinear
layer = RowParallelLinear(F * n, H, has_bias=False, input_is_parallel=True)
layer.to(dtype="bfloat16")
xr = (torch.randn(2, T // 2, F, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
wr = layer.weight
assert FL.linear_all_reduce_ok(xr.reshape(-1, F), wr, g)
yr = layer(xr)
dyr = (torch.randn(2, T // 2, H, generator=torch.Generator(device="cuda").manual_seed(5), device="cuda") * 0.1).to(torch.bfloat16)
yr.backward(dyr)
fullr = xr.detach().float().reshape(-1, F) @ wr.detach().float()
dist.all_reduce(fullr, group=g)
res["errs"]["row_ar_y"] = rel(yr.reshape(-1, H), fullr)
res["errs"]["row_ar_dx"] = rel(xr.grad.reshape(-1, F), dyr.float().reshape(-1, H) @ wr.detach().float().t())
res["errs"]["row_ar_dw"] = rel(wr.grad, xr.detach().float().reshape(-1, F).t() @ dyr.float().reshape(-1, H))
_lib.check_status()


def bench(fn, iters=20):
    for _ in range(3):
        fn()
    dist.barrier(); torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record(); torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, dist.ReduceOp.MAX)
    return float(t)


with torch.no_grad():
    xd, wd = x.detach(), w.detach()
    x2d, w2d = x2.detach(), w2.detach()
    res["t_ag_fused"] = bench(lambda: FL._AllGatherLinear.apply(xd, wd, g))
    res["t_ag_nccl"] = bench(lambda: torch.matmul(spu.all_gather(xd, g), wd))
    res["t_rs_fused"] = bench(lambda: FL._LinearReduceScatter.apply(x2d, w2d, g))
    res["t_rs_nccl"] = bench(lambda: spu.reduce_scatter(torch.matmul(x2d, w2d), g))
    res["t_gemm_only_ag"] = bench(lambda: torch.matmul(xf.to(torch.bfloat16), wd))
res["shape"] = (T, H, F, n)
_probe = FL._AGSlot(g, 128, 64)
res["multicast"] = bool(_probe.mc_stage)
res["push_mode"] = _probe.push_mode
res["rs_mc"] = bool(FL._RSSlot(g, 128, 64).mc)
_lib.check_status()
_common.dump(res)
