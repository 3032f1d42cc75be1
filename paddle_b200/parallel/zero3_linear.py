"""Sharding stage 3 linear layer whose parameter all-gather is fused into the consuming GEMM.

The weight ``W [in, out]`` is stored as row slices ``W_r [in / n, out]``.  Forward is ONE kernel: communication CTAs
push this rank's slice into every peer's staging buffer while the tensor-core CTAs already multiply the k-blocks that
have arrived (local slice first), so the gather hides under the GEMM and the full weight never exists outside the
staging buffer.  Backward re-gathers through NCCL (the reference's stage-3 behaviour: group_sharded_stage3.py
``_register_forward_hooks`` / backward re-gather), computes dX with the tcgen05 GEMM and reduce-scatters dW."""
from __future__ import annotations

import torch

from .._core.tensor import as_tensor
from ..distributed import collective as C
from ..ops import native
from . import fused_linear_impl as FL


class _Zero3LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_shard, group):
        n = group.nranks
        rows, N = w_shard.shape
        K = rows * n
        x2 = x.reshape(-1, K).contiguous()
        M = x2.shape[0]
        slot = FL._slot("ag", group, rows, N)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        FL.ag_gemm(slot, group, w_shard.detach().contiguous(), x2, slot.stage, out, M, N, K, 0, 1, 0, 1, gathered_b=True)
        ctx.save_for_backward(x2, w_shard)
        ctx.group, ctx.shape = group, x.shape
        return out.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, w_shard = ctx.saved_tensors
        group = ctx.group
        n = group.nranks
        rows, N = w_shard.shape
        dy2 = dy.reshape(-1, N).contiguous()
        full = torch.empty((rows * n, N), dtype=w_shard.dtype, device=w_shard.device)
        C.all_gather_into_tensor(full, w_shard.detach().contiguous(), group=group)
        dx = native.gemm(dy2, full, trans_b=True)
        dw_full = native.gemm(x2, dy2, trans_a=True, out_dtype=torch.float32)
        dw = torch.empty((rows, N), dtype=torch.float32, device=w_shard.device)
        C.reduce_scatter(dw, list(dw_full.chunk(n, 0)), group=group)
        return dx.view(ctx.shape), dw.to(w_shard.dtype), None


def zero3_linear(x, w_shard, group):
    """``x [.., in] @ gather_rows(w_shard)``; ``w_shard`` is this rank's ``[in / n, out]`` slice (bf16, CUDA)."""
    return as_tensor(_Zero3LinearFn.apply(x, w_shard, group))
