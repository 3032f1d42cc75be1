"""Sharding stage 3 linear layer whose parameter all-gather is fused into the consuming GEMMs.

The weight ``W [in, out]`` is stored as row slices ``W_r [in / n, out]`` (the flat 1/n slices that
``GroupShardedStage3`` keeps are exactly these when ``in % n == 0``).  The full weight never exists outside the
staging buffer of the fused kernels:

* forward   ``Y = X gather(W)``: communication CTAs push this rank's slice to every peer while the tensor-core CTAs
  already multiply the k-blocks that have arrived (tokens of the gathered matrix are the reduction dimension);
* backward  ``dX^T = gather(W) dY^T``: the slices are gathered again inside the GEMM (rows of the gathered matrix are the
  output rows, consumed in arrival order), so the re-gather of the reference's stage 3
  (python/paddle/distributed/fleet/meta_parallel/sharding/group_sharded_stage3.py:560-616 hooks, :1077-1125
  ``_allgather_buffer``) hides under the input-gradient GEMM;
* backward  ``dW_r = reduce_scatter(X^T dY)``: the weight-gradient GEMM pushes every partial tile to the rank that owns
  those rows of ``W`` and the owner reduces them (GEMM -> reduce-scatter), instead of the reference's all-reduce of the
  full gradient followed by a slice (:746-764).

Shapes the fused kernels cannot take (``in / n`` not a multiple of 128, non-bf16) go through NCCL collectives and the
plain GEMM."""
from __future__ import annotations

import torch

from .._core.tensor import as_tensor
from ..distributed import collective as C
from ..ops import native
from . import fused_linear_impl as FL


def fused_ok(w_shard, group) -> bool:
    rows, N = w_shard.shape
    return (w_shard.is_cuda and w_shard.dtype == torch.bfloat16 and rows % FL.SUB_ROWS == 0 and N % 8 == 0
            and group is not None and group.nranks in (2, 4, 8) and FL.symm.supported())


class _Zero3LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_shard, group, grad_scale):
        n = group.nranks
        rows, N = w_shard.shape
        K = rows * n
        x2 = x.reshape(-1, K).contiguous()
        M = x2.shape[0]
        ws = w_shard.detach().contiguous()
        if fused_ok(w_shard, group):
            slot = FL._slot("ag", group, rows, N)
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
            FL.ag_gemm(slot, group, ws, x2, slot.stage, out, M, N, K, 0, 1, 0, 1, gathered_b=True)
        else:
            full = torch.empty((K, N), dtype=ws.dtype, device=ws.device)
            C.all_gather_into_tensor(full, ws, group=group)
            out = native.gemm(x2, full) if x2.is_cuda and x2.dtype == torch.bfloat16 else x2 @ full
        ctx.save_for_backward(x2, w_shard)
        ctx.group, ctx.shape, ctx.grad_scale = group, x.shape, grad_scale
        return out.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, w_shard = ctx.saved_tensors
        group = ctx.group
        n = group.nranks
        rows, N = w_shard.shape
        K = rows * n
        M = x2.shape[0]
        dy2 = dy.reshape(-1, N).contiguous()
        ws = w_shard.detach().contiguous()
        dx = dw = None
        if fused_ok(w_shard, group) and M % 8 == 0:
            if ctx.needs_input_grad[0]:
                slot = FL._slot("ag", group, rows, N)
                dxT = torch.empty((K, M), dtype=torch.bfloat16, device=dy2.device)
                FL.ag_gemm(slot, group, ws, slot.stage, dy2, dxT, K, M, N, 0, 0, 0, 0)       # gather(W) dY^T
                dx = dxT.t().contiguous().view(ctx.shape)
            if ctx.needs_input_grad[1]:
                rs = FL._slot("rs", group, rows, N)
                dw = torch.empty((rows, N), dtype=torch.bfloat16, device=dy2.device)
                FL.gemm_rs(rs, group, x2, dy2, dw, K, N, M, 1, 1)                            # X^T dY -> owner of the rows
                if ctx.grad_scale != 1.0:
                    dw.mul_(ctx.grad_scale)
            return dx, dw, None, None
        full = torch.empty((K, N), dtype=ws.dtype, device=ws.device)
        C.all_gather_into_tensor(full, ws, group=group)
        gpu = dy2.is_cuda and dy2.dtype == torch.bfloat16
        if ctx.needs_input_grad[0]:
            dx = (native.gemm(dy2, full, trans_b=True) if gpu else dy2 @ full.t()).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            dw_full = native.gemm(x2, dy2, trans_a=True, out_dtype=torch.float32) if gpu else (x2.t() @ dy2).float()
            dwf = torch.empty((rows, N), dtype=torch.float32, device=ws.device)
            C.reduce_scatter(dwf, list(dw_full.chunk(n, 0)), group=group)
            dw = (dwf * ctx.grad_scale).to(w_shard.dtype)
        return dx, dw, None, None


def zero3_linear(x, w_shard, group, grad_scale=1.0):
    """``x [.., in] @ gather_rows(w_shard)``; ``w_shard`` is this rank's ``[in / n, out]`` slice.  The gradient of
    ``w_shard`` is the sum over ranks of the local weight gradients times ``grad_scale`` (1 / n for data-parallel
    averaging)."""
    return as_tensor(_Zero3LinearFn.apply(x, w_shard, group, grad_scale))
