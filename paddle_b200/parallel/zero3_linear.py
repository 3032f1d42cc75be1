"""Sharding stage 3 linear layer whose parameter all-gather is fused into the consuming GEMMs.

The weight ``W [in, out]`` is stored as row slices ``W_r [in / n, out]`` (the flat 1/n slices that
``GroupShardedStage3`` keeps are exactly these when ``in % n == 0``).  The full weight never exists outside the
staging buffer of the fused kernels:

* forward   ``Y = X gather(W)``: by default the slices are gathered one layer ahead on a side stream
  (``_WeightPrefetcher``) and the product is a plain 2-CTA GEMM; with ``PD_ZERO3_FWD=fused`` communication CTAs push this
  rank's slice to every peer while the tensor-core CTAs already multiply the k-blocks that have arrived (the rows of the
  gathered matrix are the reduction dimension) - correct, but measured 2.3x slower than gather + GEMM;
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


class _WeightPrefetcher:
    """Forward-pass weight gathers one layer ahead, on a side stream.

    The stage-3 linears of a model run in the same order every iteration.  The first forward pass records that order;
    from then on, when linear i starts, the all-gather of linear i+1's weight slices is issued on a side stream, so it
    runs under linear i's GEMM and the GEMM of i+1 finds the full weight waiting (the reference prefetches the same way
    around its forward hooks: group_sharded_stage3.py ``_forward_pre_hook`` / ``_allgather_buffer`` :1077-1125).  The
    consumer is then a plain 2-CTA GEMM at its full rate.  Measured on two GPUs for the 7B qkv shape (4096 tokens,
    4096 x 12288): all-gather fused into the K-gathered GEMM kernel 914 us, NCCL all-gather followed by the GEMM 397 us
    (exposed gather included), plain GEMM alone ~270 us - so the overlapped form is the default
    (``PD_ZERO3_FWD=fused`` selects the in-kernel gather).

    Buffers: a gathered weight lives in a buffer taken from a small free list keyed by size; after its GEMM the buffer
    goes back with an event, and the side stream waits for that event before it overwrites the buffer."""

    def __init__(self):
        self.order, self.pos = [], {}
        self.frozen = False
        self.stream = None
        self.pending = {}            # key -> (buffer, ready event)
        self.free = {}               # nbytes -> [(buffer, last-use event)]
        self.shards = {}             # key -> (view of the shard's storage, group)

    def _buffer(self, rows_full, N, dtype, device):
        key = (rows_full, N, dtype)
        lst = self.free.setdefault(key, [])
        if lst:
            return lst.pop(0)
        return torch.empty((rows_full, N), dtype=dtype, device=device), None

    def _issue(self, key):
        ws, group = self.shards[key]
        if key in self.pending:
            return
        if self.stream is None:
            self.stream = torch.cuda.Stream()
        n = group.nranks
        buf, last_use = self._buffer(ws.shape[0] * n, ws.shape[1], ws.dtype, ws.device)
        now = torch.cuda.Event()
        now.record()                                   # the slices may have just been updated on the compute stream
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(now)
            if last_use is not None:
                self.stream.wait_event(last_use)
            C.all_gather_into_tensor(buf, ws.detach(), group=group)
            ready = torch.cuda.Event()
            ready.record()
        self.pending[key] = (buf, ready)

    def take(self, w_shard, group):
        """Full weight of ``w_shard`` for the forward GEMM (waits for its gather), and the prefetch of the next one."""
        # the caller hands in a fresh view of the persistent slice every time: the storage address identifies the layer,
        # and the view kept here shares that storage (the optimizer updates it in place)
        key = (w_shard.data_ptr(), tuple(w_shard.shape))
        if key not in self.shards:
            self.shards[key] = (w_shard.detach(), group)
        if not self.frozen:
            if key in self.pos:                        # second visit: the order of one pass is known
                self.frozen = True
            else:
                self.pos[key] = len(self.order)
                self.order.append(key)
        if key not in self.pending:
            self._issue(key)
        buf, ready = self.pending.pop(key)
        torch.cuda.current_stream().wait_event(ready)
        # no wrap-around: between the last linear of one pass and the first of the next lie the backward pass and the
        # optimizer update of the slices, so the first layer of a pass gathers on demand
        if self.frozen and key in self.pos and self.pos[key] + 1 < len(self.order):
            self._issue(self.order[self.pos[key] + 1])
        return buf

    def give_back(self, buf):
        ev = torch.cuda.Event()
        ev.record()
        self.free.setdefault((buf.shape[0], buf.shape[1], buf.dtype), []).append((buf, ev))


_prefetcher = _WeightPrefetcher()


def _fwd_mode():
    import os
    return os.environ.get("PD_ZERO3_FWD", "prefetch")


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
        if fused_ok(w_shard, group) and _fwd_mode() == "prefetch" and not torch.cuda.is_current_stream_capturing():
            full = _prefetcher.take(w_shard, group)
            out = native.gemm(x2, full)
            _prefetcher.give_back(full)
        elif fused_ok(w_shard, group):
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
