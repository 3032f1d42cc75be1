"""Fused expert-parallel MoE (fp8-quantising dispatch over peer memory, grouped block-scaled GEMMs, weighted combine)
against the same layer on the NCCL all-to-all path, forward and backward, two steps in a row: ragged token counts per
rank, one expert that receives no token."""
import os

import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200.incubate.distributed.models.moe import MoELayer
from paddle_b200.incubate.distributed.models.moe.fp8_experts import FP8GroupedExperts
from paddle_b200.ops import _lib

dist.init_parallel_env()
rank, n = dist.get_rank(), dist.get_world_size()
group = dist.new_group(list(range(n)))
H, I, NL = 256, 512, 2
torch.manual_seed(5)


def build():
    paddle.seed(20 + rank)
    ex = FP8GroupedExperts(NL, H, I, initializer_range=0.05).to("gpu").to(dtype="bfloat16")
    paddle.seed(9)
    layer = MoELayer(H, ex, gate={"type": "naive", "top_k": 2}, moe_group=group)
    layer.to("gpu")
    layer.to(dtype="bfloat16")
    return layer


fused, plain = build(), build()
plain.set_state_dict({k: v.clone() for k, v in fused.state_dict().items()})
gw = [p for p in fused.gate.parameters() if p.dim() == 2][0]
with torch.no_grad():                     # the last global expert is never chosen
    for layer in (fused, plain):
        w = [p for p in layer.gate.parameters() if p.dim() == 2][0]
        col = w.shape[1] - 1
        w[:, col] = 0
        b = [p for p in layer.gate.parameters() if p.dim() == 1]
        if b:
            b[0][col] = -50.0
fused.fused_capacity = 512
plain._use_fused = lambda inp: False
res = {"errs": {}}


def rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))


T = 200 + 128 * rank
for step in range(2):
    x0 = (torch.randn(T, H, device="cuda") * 0.5).to(torch.bfloat16)
    outs = []
    for layer in (fused, plain):
        x = paddle.to_tensor(x0.clone()); x.stop_gradient = False
        y = layer(x)
        (y.float() ** 2).sum().backward()
        outs.append((y.detach(), x.grad.detach().clone(), [p.grad.detach().clone() for p in layer.parameters()]))
        for p in layer.parameters():
            p.grad = None
    torch.cuda.synchronize()
    _lib.check_status()
    (yf, dxf, gf), (yp, dxp, gp) = outs
    res["errs"][f"y_{step}"] = rel(yf, yp)
    res["errs"][f"dx_{step}"] = rel(dxf, dxp)
    for i, (a, b) in enumerate(zip(gf, gp)):
        res["errs"][f"dparam{i}_{step}"] = rel(a, b)
res["used_fused"] = bool(fused._use_fused(x))
res["y_absmax"] = float(yp.float().abs().max())
_common.dump(res)
