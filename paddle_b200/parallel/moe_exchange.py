"""Host side of the fused expert-parallel exchange (``csrc/kernels/moe_dispatch.cu``): symmetric receive buffers,
device-side routing metadata (no host synchronisation anywhere) and the autograd function that runs one MoE expert
block - dispatch with fp8 quantisation, the two grouped block-scaled GEMMs around SwiGLU, weighted combine - forward
and backward.

The reference path is ``MoEScatter`` / ``MoEGather`` around ``global_scatter`` / ``global_gather``
(python/paddle/incubate/distributed/models/moe/moe_layer.py:99-258), whose counts go through the host
(paddle/phi/kernels/gpu/global_scatter_kernel.cu:57-75).
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib, native
from ..ops._lib import c_int, check, ptr, stream
from . import symm

U64x8 = ctypes.c_ulonglong * 8
WAIT_MS = 4000


def _arr(vals):
    return U64x8(*(list(vals) + [0] * (8 - len(vals))))


def routing_slots(expert_idx, n_experts):
    """``expert_idx`` int ``[T, k]`` (global expert of every routed copy, negative = pruned) -> (``slot`` int32
    ``[T * k]``: position of the copy among this rank's copies for the same expert, in token order; ``counts`` int32
    ``[n_experts]``).  Device ops only."""
    flat = expert_idx.reshape(-1).to(torch.int64)
    n = flat.numel()
    key = torch.where(flat >= 0, flat, torch.full_like(flat, n_experts))
    order = torch.argsort(key, stable=True)
    counts = torch.bincount(key, minlength=n_experts + 1)
    starts = torch.cumsum(counts, 0) - counts
    rank_sorted = torch.arange(n, device=flat.device) - starts[key[order]]
    slot = torch.empty(n, dtype=torch.int64, device=flat.device)
    slot[order] = rank_sorted
    return slot.to(torch.int32), counts[:n_experts].to(torch.int32)


class MoEExchange:
    """Symmetric buffers of one (group, local experts, hidden, capacity) shape.  One object serves every MoE layer of
    that shape, forward and backward: a dispatch and the combine that follows it act as a barrier pair over the group."""

    def __init__(self, group, n_local_experts, hidden, cap):
        n = group.nranks
        assert hidden % 128 == 0 and n_local_experts * n <= 64
        self.group, self.n, self.E_local, self.H, self.cap = group, n, n_local_experts, hidden, int(cap)
        self.n_seg = n_local_experts * n
        self.M_pad = self.n_seg * self.cap
        nb = hidden // 128

        def al(v):
            return (v + 255) // 256 * 256
        self.off_xq = 0
        self.off_xs = al(self.M_pad * hidden)
        self.off_y = self.off_xs + al(self.M_pad * nb * 4)
        self.off_counts = self.off_y + al(self.M_pad * hidden * 2)
        self.off_ready = self.off_counts + al(self.n_seg * 4)
        self.off_oready = self.off_ready + 256
        self.block = symm.SymmBlock(self.off_oready + 256, group)
        b = self.block
        self.xq = b.view(self.off_xq, (self.M_pad, hidden), torch.uint8).view(torch.float8_e4m3fn)
        self.xs = b.view(self.off_xs, (self.M_pad, nb), torch.float32)
        self.y = b.view(self.off_y, (self.M_pad, hidden), torch.bfloat16)
        self.p_xq, self.p_xs = _arr(b.peer_ptrs(self.off_xq)), _arr(b.peer_ptrs(self.off_xs))
        self.p_y, self.p_counts = _arr(b.peer_ptrs(self.off_y)), _arr(b.peer_ptrs(self.off_counts))
        self.p_ready, self.p_oready = _arr(b.peer_ptrs(self.off_ready)), _arr(b.peer_ptrs(self.off_oready))
        dev = b.local.device
        self.state_d = torch.zeros(2, dtype=torch.int32, device=dev)
        self.state_c = torch.zeros(2, dtype=torch.int32, device=dev)
        self.seg_start = torch.zeros(self.n_seg, dtype=torch.int32, device=dev)
        self.seg_end = torch.zeros(self.n_seg, dtype=torch.int32, device=dev)
        self.expert_map = torch.zeros(self.n_seg, dtype=torch.int32, device=dev)
        self._row_seg = (torch.arange(self.M_pad, device=dev) // self.cap)
        self._row_pos = (torch.arange(self.M_pad, device=dev) % self.cap).to(torch.int32)

    # ------------------------------------------------------------------ kernels
    def dispatch(self, x, expert, slot, send_counts, row_scale=None):
        """Quantise and push every routed copy of ``x [T, H]`` to the owner of its expert; on return (stream order) this
        rank's ``xq`` / ``xs`` hold the rows it received and ``seg_start`` / ``seg_end`` / ``expert_map`` describe them."""
        T, H = x.shape
        k = expert.numel() // T
        rc = _lib.kernels().pd_moe_dispatch_fp8(
            ptr(x), ptr(expert), ptr(slot), ptr(row_scale), ptr(send_counts), c_int(T), c_int(k), c_int(H), c_int(self.cap),
            c_int(self.E_local), c_int(self.group.rank), c_int(self.n), self.p_xq, self.p_xs, self.p_counts, self.p_ready,
            ptr(self.state_d), ptr(self.seg_start), ptr(self.seg_end), ptr(self.expert_map), c_int(WAIT_MS),
            ptr(_lib.status_buffer(x.device)), stream())
        check(rc, "pd_moe_dispatch_fp8")
        native._count()

    def combine(self, expert, slot, T, weight=None, want_rows=False):
        """Gather every token's expert rows from the owners' ``y`` buffers and sum them (times ``weight``)."""
        k = expert.numel() // T
        out = torch.empty((T, self.H), dtype=torch.bfloat16, device=self.y.device)
        rows = torch.empty((T * k, self.H), dtype=torch.bfloat16, device=self.y.device) if want_rows else None
        rc = _lib.kernels().pd_moe_combine(
            ptr(expert), ptr(slot), ptr(weight), ptr(out), ptr(rows), c_int(T), c_int(k), c_int(self.H), c_int(self.cap),
            c_int(self.E_local), c_int(self.group.rank), c_int(self.n), self.p_y, self.p_oready, ptr(self.state_c),
            c_int(WAIT_MS), ptr(_lib.status_buffer(out.device)), stream())
        check(rc, "pd_moe_combine")
        native._count()
        return out, rows

    def grouped(self, a_q, a_s, w_q, w_s, out):
        """``out[rows of segment s] = a[rows] @ W[expert_map[s]]`` over the segments of the last dispatch."""
        M, K = a_q.shape
        E_w, N, _ = w_q.shape
        max_tiles = self.n_seg * ((self.cap + 127) // 128) * (N // 128)
        rc = _lib.kernels().pd_grouped_gemm_fp8_seg(
            ptr(a_q), ptr(a_s), ptr(w_q), ptr(w_s), ptr(self.seg_start), ptr(self.seg_end), ptr(self.expert_map), ptr(out),
            c_int(M), c_int(N), c_int(K), c_int(self.n_seg), c_int(E_w), c_int(out.stride(0)), c_int(max_tiles),
            ptr(_lib.status_buffer(out.device)), stream())
        check(rc, "pd_grouped_gemm_fp8_seg")
        native._count()
        return out

    # ------------------------------------------------------------------ helpers (device ops, no sync)
    def valid_rows(self):
        """bool ``[M_pad]``: rows of the receive buffers that hold a token of the last dispatch."""
        counts = (self.seg_end - self.seg_start)
        return self._row_pos < counts[self._row_seg]

    def received_bf16(self, valid):
        """The received rows dequantised to bf16, unused rows zero (operand of the weight-gradient GEMMs)."""
        nb = self.H // 128
        v = self.xq.float().view(self.M_pad, nb, 128) * self.xs.view(self.M_pad, nb, 1)
        v = torch.where(valid.view(-1, 1, 1), v, torch.zeros((), device=v.device))
        return v.view(self.M_pad, self.H).to(torch.bfloat16)


_exchanges = {}


def get_exchange(group, n_local_experts, hidden, cap):
    key = (group.id, n_local_experts, hidden, int(cap))
    ex = _exchanges.get(key)
    if ex is None:
        ex = MoEExchange(group, n_local_experts, hidden, cap)
        _exchanges[key] = ex
    return ex


class _FusedMoEFn(torch.autograd.Function):
    """One expert block of an expert-parallel MoE layer.

    forward:  dispatch (quantise + push) -> grouped fp8 GEMM with ``w1`` -> SwiGLU -> quantise -> grouped fp8 GEMM with
              ``w2`` into the symmetric output buffer -> combine (pull + gate-weighted sum)
    backward: the mirror - ``gate * dout`` is dispatched (the gate value is folded into the quantisation), the two
              input-gradient GEMMs run on the transposed e4m3 weights, the expert input gradients return through the
              combine kernel (plain sum over the k copies); weight gradients are bf16 tcgen05 GEMMs over each local
              expert's receive region (unused rows are zero), accumulated into ``main_grad`` when present.
    ``x [T, H]`` bf16, ``gate_w [T, k]`` fp32, ``w1 [E_local, H, 2 I]``, ``w2 [E_local, I, H]`` bf16."""

    @staticmethod
    def forward(ctx, x, gate_w, w1, w2, ex, expert, slot, send_counts, caches):
        x = x.contiguous()
        T, H = x.shape
        gw = gate_w.detach().reshape(-1).float().contiguous()
        ex.dispatch(x, expert, slot, send_counts)
        valid = ex.valid_rows()
        need_w = w1.requires_grad or w2.requires_grad
        xd = ex.received_bf16(valid) if need_w else None
        w1q, w1s = caches[0].get(w1, False)
        w2q, w2s = caches[1].get(w2, False)
        h = torch.zeros((ex.M_pad, w1.shape[2]), dtype=torch.bfloat16, device=x.device)
        ex.grouped(ex.xq, ex.xs, w1q, w1s, h)
        a = native.swiglu_fwd(h)
        aq, as_ = native.fp8_quant_1x128(a)
        ex.grouped(aq, as_, w2q, w2s, ex.y)
        out, rows = ex.combine(expert, slot, T, weight=gw, want_rows=True)
        ctx.save_for_backward(xd, h, rows, gw, expert, slot, send_counts, w1, w2)
        ctx.ex, ctx.caches, ctx.shape_gate = ex, caches, gate_w.shape
        ctx.w_refs = (w1, w2)
        return out

    @staticmethod
    def backward(ctx, dout):
        xd, h, rows, gw, expert, slot, send_counts, w1, w2 = ctx.saved_tensors
        ex, caches = ctx.ex, ctx.caches
        dout = dout.contiguous()
        T, H = dout.shape
        k = gw.numel() // T
        d_gate = None
        if ctx.needs_input_grad[1]:
            d_gate = (rows.view(T, k, H).float() * dout.view(T, 1, H).float()).sum(-1).view(ctx.shape_gate)
        # gate-weighted output gradient to the experts (fp8 for the input-gradient GEMM, bf16 for the weight gradient)
        ex.dispatch(dout, expert, slot, send_counts, row_scale=gw)
        valid = ex.valid_rows()
        need_w = ctx.needs_input_grad[2] or ctx.needs_input_grad[3]
        dyd = ex.received_bf16(valid) if need_w else None
        a = native.swiglu_fwd(h)
        w2tq, w2ts = caches[1].get(w2, True)
        da = torch.zeros((ex.M_pad, w2.shape[1]), dtype=torch.bfloat16, device=dout.device)
        ex.grouped(ex.xq, ex.xs, w2tq, w2ts, da)
        dh, _ = native.swiglu_bwd(h, None, da)
        dw1 = dw2 = None
        if need_w:
            dw1, dw2 = _weight_grads(ctx.w_refs, xd, dh, a, dyd, ex)
        dhq, dhs = native.fp8_quant_1x128(dh)
        w1tq, w1ts = caches[0].get(w1, True)
        ex.grouped(dhq, dhs, w1tq, w1ts, ex.y)
        dx, _ = ex.combine(expert, slot, T, weight=None)
        return dx, d_gate, dw1, dw2, None, None, None, None, None


def _weight_grads(w_refs, xd, dh, a, dyd, ex):
    """dW1[e] (+)= X_e^T dH_e and dW2[e] (+)= A_e^T dY_e over each local expert's receive region."""
    w1, w2 = w_refs
    rows_e = ex.n * ex.cap
    outs = []
    for w, lhs, rhs in ((w1, xd, dh), (w2, a, dyd)):
        mg = getattr(w, "main_grad", None)
        dw = None if mg is not None else torch.empty_like(w)
        for e in range(ex.E_local):
            sl = slice(e * rows_e, (e + 1) * rows_e)
            if mg is not None:
                native.gemm(lhs[sl], rhs[sl], trans_a=True, out=mg[e], accumulate=True)
            else:
                native.gemm(lhs[sl], rhs[sl], trans_a=True, out=dw[e])
        if mg is not None:
            hook = getattr(w, "_main_grad_ready_hook", None)
            if hook is not None:
                hook(w)
        outs.append(dw)
    return outs


def fused_moe_available(x, experts, group) -> bool:
    """GPU, bf16, stacked (grouped) fp8 experts, a group of up to 8 ranks with symmetric memory."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and getattr(experts, "grouped", False)):
        return False
    import os
    if os.environ.get("PD_FUSED_MOE", "1") == "0":          # comparison arm: NCCL all-to-all dispatch / combine
        return False
    if group is None or group.nranks > 8 or not symm.supported():
        return False
    from ..ops import functional as K
    if K.get_kernel_policy() != "fused":
        return False
    w1, w2 = experts.gate_up_weight, experts.down_weight
    return (w1.dtype == torch.bfloat16 and x.shape[-1] % 128 == 0 and w1.shape[2] % 256 == 0 and w2.shape[1] % 128 == 0)


def fused_moe_forward(x, gate_value, gate_idx, experts, group, capacity_factor=1.25, cap=None):
    """``x [T, H]``; ``gate_value`` / ``gate_idx`` ``[T, k]`` from the router (index < 0 = pruned).  Copies beyond the
    per-(expert, source rank) capacity ``ceil(capacity_factor * k * T / n_experts)`` (rounded up to 128) are dropped."""
    T, H = x.shape
    k = gate_idx.shape[1] if gate_idx.dim() > 1 else 1
    n_exp = experts.num_experts * group.nranks
    if cap is None:
        cap = int(-(-capacity_factor * k * T // n_exp))
    cap = max(128, (int(cap) + 127) // 128 * 128)
    ex = get_exchange(group, experts.num_experts, H, cap)
    idx = torch.as_tensor(gate_idx).reshape(T, k)
    slot, counts = routing_slots(idx, n_exp)
    expert = idx.reshape(-1).to(torch.int32).contiguous()
    return _FusedMoEFn.apply(x, gate_value, experts.gate_up_weight, experts.down_weight, ex, expert, slot, counts,
                             experts._cache)
