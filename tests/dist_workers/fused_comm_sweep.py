"""Timing sweep of the fused comm GEMMs (diagnostic; prints from rank 0)."""
import os
import sys

import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200.distributed import fleet
from paddle_b200.ops import _lib, native

os.environ["PD_AG_COMM_CTAS"] = "8"          # the sweep sets FL.N_COMM itself
n = int(os.environ["PADDLE_TRAINERS_NUM"])
strategy = fleet.DistributedStrategy()
strategy.hybrid_configs = {"dp_degree": 1, "mp_degree": n}
fleet.init(is_collective=True, strategy=strategy)
rank = dist.get_rank()
g = fleet.get_hybrid_communicate_group().get_model_parallel_group()
from paddle_b200.parallel import fused_linear_impl as FL
from paddle_b200.distributed.fleet.utils import sequence_parallel_utils as spu


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


T, H = 4096, 4096
res = {}
for name, Ncol, Krow in (("qkv", 3 * H // n, H // n), ("gate_up", 2 * 11008 // n // 8 * 8, 11008 // n // 8 * 8)):
    rows = T // n
    x = torch.randn(rows, H, device="cuda").to(torch.bfloat16)
    w = (torch.randn(H, Ncol, device="cuda") * 0.05).to(torch.bfloat16)
    xfull = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    x2 = torch.randn(T, Krow, device="cuda").to(torch.bfloat16)
    w2 = (torch.randn(Krow, H, device="cuda") * 0.05).to(torch.bfloat16)
    with torch.no_grad():
        res[f"{name}_plain_gemm_colshape"] = bench(lambda: native.gemm(xfull, w))
        res[f"{name}_plain_gemm_rowshape"] = bench(lambda: native.gemm(x2, w2))
        res[f"{name}_cublas_colshape"] = bench(lambda: torch.matmul(xfull, w))
        res[f"{name}_cublas_rowshape"] = bench(lambda: torch.matmul(x2, w2))
        res[f"{name}_nccl_ag"] = bench(lambda: spu.all_gather(x, g))
        res[f"{name}_nccl_rs"] = bench(lambda: spu.reduce_scatter(torch.empty(T, H, device="cuda", dtype=torch.bfloat16), g))
        for nc in (4, 8, 16, 32):
            FL.N_COMM = nc
            FL._slots.clear()
            res[f"{name}_ag_fused_comm{nc}"] = bench(lambda: FL._AllGatherLinear.apply(x, w, g))
        FL.N_COMM = 8
        FL._slots.clear()
        slot = FL._slot("ag", g, rows, H)
        y = torch.empty(T, Ncol, device="cuda", dtype=torch.bfloat16)
        FL.ag_gemm(slot, g, x, slot.stage, w, y, T, Ncol, H, 0, 1, 0, 0)
        dist.barrier(); torch.cuda.synchronize()
        res[f"{name}_ag_gemm_only_nopush"] = bench(
            lambda: FL.ag_gemm(slot, g, x, slot.stage, w, y, T, Ncol, H, 0, 1, 0, 0, push=False, ack=False))
        res[f"{name}_ag_nopush_plainA"] = bench(
            lambda: FL.ag_gemm(slot, g, x, xfull, w, y, T, Ncol, H, 0, 1, 0, 0, push=False, ack=False))
        res[f"{name}_plain_gemm_140ctas"] = bench(lambda: native.gemm(xfull, w, max_ctas=140))
        FL.N_COMM = 0
        FL._slots.clear()
        slot0 = FL._slot("ag", g, rows, H)
        slot0.epoch = 0
        res[f"{name}_ag_nopush_comm0"] = bench(
            lambda: FL.ag_gemm(slot0, g, x, xfull, w, y, T, Ncol, H, 0, 1, 0, 0, push=False, ack=False))
        FL.N_COMM = 8
        res[f"{name}_rs_fused"] = bench(lambda: FL._LinearReduceScatter.apply(x2, w2, g))
_lib.check_status()
if rank == 0:
    for k, v in res.items():
        print(f"{k:40s} {v * 1000:9.1f} us", flush=True)
_common.dump(res)
