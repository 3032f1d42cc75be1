"""Host side of the fused all-gather->GEMM / GEMM->reduce-scatter kernels: symmetric staging slots,
epoch bookkeeping and the autograd functions behind the sequence-parallel linears."""
from __future__ import annotations

import ctypes
import os

import torch

from .._core.tensor import as_tensor
from ..ops import _lib, native
from ..ops._lib import c_int, check, ptr, stream
from . import symm

BM, BN = 128, 256
SUB_ROWS = 128
N_COMM = int(os.environ.get("PD_AG_COMM_CTAS", "8"))
WAIT_MS = int(os.environ.get("FLAGS_pd_wait_limit_ms", "2000"))
_slots = {}
_sm_count = None
U64x8 = ctypes.c_ulonglong * 8


def _sms():
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def _arr(vals):
    return U64x8(*(list(vals) + [0] * (8 - len(vals))))


def _env_int(name, default):
    v = os.environ.get(name)
    return default if v is None or v == "" else int(v)


PARTS = 8            # push jobs per 128-row chunk (vector / multicast push); a chunk's flag counts to epoch * PARTS


class _AGSlot:
    """Staging for one gathered matrix [nranks * rows, row_elems] bf16 + arrival counters + acks.

    ``push_mode``: 2 = multimem.st through the block's multicast address (NVLS), 1 = 16-byte stores to every peer
    from all threads of the push CTAs, 0 = bulk-copy ring driven by one thread per push CTA.  The default is 2
    where the fabric offers multicast, else 1; ``PD_AG_PUSH_MODE`` overrides (a slot keeps its mode for life:
    the arrival counters count ``parts`` pushes per chunk and epoch)."""

    def __init__(self, group, rows, row_elems):
        n = group.nranks
        self.n, self.rows, self.row_elems = n, rows, row_elems
        self.n_sub = rows // SUB_ROWS
        stage_bytes = n * rows * row_elems * 2
        self.off_flags = (stage_bytes + 255) // 256 * 256
        self.off_ack = self.off_flags + ((n * self.n_sub * 4 + 255) // 256 * 256)
        self.block = symm.SymmBlock(self.off_ack + 256, group)
        self.stage = self.block.view(0, (n * rows, row_elems), torch.bfloat16)
        self.p_stage = _arr(self.block.peer_ptrs(0))
        self.p_flags = _arr(self.block.peer_ptrs(self.off_flags))
        self.p_ack = _arr(self.block.peer_ptrs(self.off_ack))
        self.mc_stage = self.block.mc_ptr
        # two ranks: one peer, the bulk-copy ring already hides the 16 MB under the local half of the GEMM (measured:
        # 306 us ring / 324 us vector / 343 us multicast for the gate_up shape)
        mode = _env_int("PD_AG_PUSH_MODE", 0 if n == 2 else (2 if self.mc_stage else 1))
        if mode == 2 and not self.mc_stage:
            mode = 1
        self.push_mode = mode
        self.parts = PARTS if mode != 0 else 1
        self.done = torch.zeros(1, dtype=torch.int32, device=self.stage.device)
        self.epoch = 0
        self.done_base = 0
        self.pending_backward = False     # staged data is still owed to a backward pass (deferred acknowledgement)
        _init_bias(self, self.stage.device)


class _RSSlot:
    """Receive buffer [nranks][rows][N] bf16 + per-tile arrival counters + acks."""

    mc = False

    def __init__(self, group, rows, N):
        n = group.nranks
        self.n, self.rows, self.N = n, rows, N
        tiles = ((rows + BM - 1) // BM) * ((N + BN - 1) // BN)
        recv_bytes = n * rows * N * 2
        self.off_cnt = (recv_bytes + 255) // 256 * 256
        self.off_ack = self.off_cnt + ((tiles * 4 + 255) // 256 * 256)
        self.block = symm.SymmBlock(self.off_ack + 256, group)
        self.p_recv = _arr(self.block.peer_ptrs(0))
        self.p_cnt = _arr(self.block.peer_ptrs(self.off_cnt))
        self.p_ack = _arr(self.block.peer_ptrs(self.off_ack))
        self.mc_partial = self.block.mc_ptr
        # with a multicast mapping the same block holds this rank's full partial product [nranks * rows, N] and the
        # owner of a slab reads it with multimem.ld_reduce (gemm_rs_mc); the layout has the same size either way
        # Opt-in (``PD_RS_MODE=1``): measured in isolation the push form is the faster one - o_proj / down shapes of
        # the 7B model 117 against 135 us on two ranks, 79 / 111 against 113 / 153 us on four - because the reducers
        # pull through latency-bound ld_reduce loads (a reducer SM sustains a few GB/s of reduced rows) and every
        # reducer is an SM taken from the GEMM.
        self.mc = bool(self.mc_partial) and _env_int("PD_RS_MODE", 0) == 1
        self.n_red = _env_int("PD_RS_RED_CTAS", 32)
        self.done = torch.zeros(1, dtype=torch.int32, device=self.block.local.device)
        self.epoch = 0
        self.done_base = 0
        _init_bias(self, self.block.local.device)


def _init_bias(slot, device):
    """Device int[2] added by the kernels to the {epoch, done_target} arguments.  Eager launches pass
    ``value - bias_host`` so the sum is the true value; a captured launch keeps its constant arguments and every
    replay of the graph ends by adding the graph's per-replay advance to ``bias`` (see :class:`GraphCapture`)."""
    slot.bias = torch.zeros(2, dtype=torch.int32, device=device)
    slot.bias_host = [0, 0]


def _slot(kind, group, rows, width):
    """Two alternating slots per (group, kind, shape) so consecutive calls rarely wait for an ack."""
    key = (group.id, kind, rows, width)
    pair = _slots.get(key)
    if pair is None:
        cls = _AGSlot if kind == "ag" else _RSSlot
        pair = {"slots": [cls(group, rows, width), cls(group, rows, width)], "next": 0}
        _slots[key] = pair
    s = pair["slots"][pair["next"]]
    pair["next"] ^= 1
    return s


KEEP_GATHERED = _env_int("PD_AG_KEEP_GATHERED", 1)
_KEEP_MAX_SLOTS = 4          # per weight: forwards in flight before their backward (pipeline schedules)
_OWNED_TOTAL_MAX = 512       # overall cap on weight-owned staging slots; beyond it backward gathers again
_owned_total = 0


def _owned_slot(group, rows, width, owner):
    """A staging slot that belongs to one weight: the matrix gathered in forward stays staged until that layer's
    weight-gradient GEMM has read it, so backward does not gather the activation a second time (32 MB per layer
    at hidden 4096, which 180 GB of HBM affords).  Returns None when every slot of the owner is still owed to a
    backward pass (several forwards in flight, as in a pipeline schedule): the caller then uses a shared slot and
    backward gathers again."""
    key = (group.id, "agw", rows, width, id(owner))
    ring = _slots.get(key)
    if ring is None:
        ring = {"slots": [], "next": 0}
        _slots[key] = ring
    for s in ring["slots"]:
        if not s.pending_backward:
            return s
    global _owned_total
    if len(ring["slots"]) < _KEEP_MAX_SLOTS and _owned_total < _OWNED_TOTAL_MAX and not _capturing():
        _owned_total += 1
        s = _AGSlot(group, rows, width)
        ring["slots"].append(s)
        return s
    return None


def _capturing():
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


class GraphCapture:
    """Bookkeeping that lets launches of the fused communication kernels sit inside a CUDA graph.

    Every slot's epoch (and acknowledgement count) must keep growing across replays although a captured launch has
    constant arguments.  ``begin()`` notes the counters, ``end_capture()`` (still inside the capture) records one
    ``bias += delta`` per slot as the last node of the graph, ``finish()`` (after the capture) computes each slot's
    advance per replay, stores it in ``delta`` and rolls the host counters back (capturing launches nothing), and
    ``replayed()`` advances the host mirrors after each replay so eager launches and other graphs stay in step."""

    def __init__(self):
        self._slots = [s for pair in _slots.values() for s in pair["slots"]]
        self._next = {k: pair["next"] for k, pair in _slots.items()}
        self._before = [(s.epoch, s.done_base) for s in self._slots]
        self._delta = [torch.zeros(2, dtype=torch.int32, device=s.bias.device) for s in self._slots]
        self._adv = None
        self._n_keys = len(_slots)

    def end_capture(self):
        if len(_slots) != self._n_keys:
            raise RuntimeError("a fused-communication slot was created during CUDA-graph capture; run the captured "
                               "code once eagerly first so that all symmetric buffers exist")
        for s, d in zip(self._slots, self._delta):
            s.bias.add_(d)

    def finish(self):
        self._adv = []
        for s, (e0, d0), d in zip(self._slots, self._before, self._delta):
            adv = (s.epoch - e0, s.done_base - d0)
            self._adv.append(adv)
            s.epoch, s.done_base = e0, d0
            d.copy_(torch.tensor(adv, dtype=torch.int32))
        for k, nxt in self._next.items():
            _slots[k]["next"] = nxt

    def replayed(self):
        for s, (de, dd) in zip(self._slots, self._adv):
            s.epoch += de
            s.done_base += dd
            s.bias_host[0] += de
            s.bias_host[1] += dd


def available(x, weight, group=None) -> bool:
    if not symm.supported() or group is None or group.nranks not in (2, 4, 8):
        return False
    if os.environ.get("PD_DISABLE_FUSED_COMM") == "1":
        return False
    return x.dim() == 2 and x.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0


def _ag_ok(rows):
    return rows % SUB_ROWS == 0


_COMM_BASE = {2: 8, 4: 16, 8: 24}          # bulk-copy ring (push_mode 0)
_COMM_VEC = {2: 8, 4: 16, 8: 28}           # vector stores to every peer (push_mode 1): n - 1 stores per 16 bytes
_COMM_MC = {2: 8, 4: 16, 8: 16}             # multicast stores (push_mode 2): one store per 16 bytes


PUSH_BYTES_PER_US_PER_CTA = 13e3     # measured: one SM sustains 12-15 GB/s of NVLink stores (any push form)
GEMM_FLOP_PER_US_PER_SM = 8.5e6      # 1-CTA tile loop of the fused kernels under load (~1250 TFLOP/s over 148 SMs)


def _comm_ctas(nranks, tiles, jobs, push, mode=0, work=None):
    """CTAs that push the local shard to the peers.  ``PD_AG_COMM_CTAS`` overrides.

    The launch ends at about max(GEMM time on the remaining SMs, push time + a short tail), because tiles are visited
    in arrival order and only the last chunks' tiles have to wait for the end of the push.  With ``work`` =
    (M, N, K, bytes this rank must send) the count that balances the two is chosen: a small GEMM behind a full-size
    gather (the dgrad of a row-parallel layer: 69 GFLOP behind 16 MB on 2 GPUs) needs twice the push CTAs of a large one,
    or it spends its time waiting for data at 8 x 13 GB/s.  Bounds: the per-degree table value halved from below, the
    number of push jobs and 64 from above.  Without ``work`` the table value is used (plus, on 4+ ranks, the SMs the
    GEMM's last wave cannot fill).  A launch that does not push has no communication CTAs at all."""
    if not push:
        return 0
    if "PD_AG_COMM_CTAS" in os.environ:
        return max(1, min(N_COMM, jobs))
    table = (_COMM_BASE, _COMM_VEC, _COMM_MC)[mode]
    base = min(table.get(nranks, 8), max(jobs, 1))
    sms = _sms()
    if work is not None and os.environ.get("PD_AG_COMM_MODEL", "1") != "0":
        M, N, K, send_bytes = work
        tile_us = 2.0 * BM * BN * K / GEMM_FLOP_PER_US_PER_SM
        best, best_t = base, None
        for c in range(max(2, base // 2), min(max(jobs, 1), 64) + 1):
            waves = -(-tiles // (sms - c))
            gemm_us = waves * tile_us
            push_us = send_bytes / (c * PUSH_BYTES_PER_US_PER_CTA) + 8.0 + tile_us
            t = max(gemm_us, push_us)
            if best_t is None or t < best_t - 0.5:
                best, best_t = c, t
        return best
    if nranks < 4 or mode == 2:
        return base
    waves = -(-tiles // (sms - base))
    needed = -(-tiles // waves)
    return max(base, min(sms - needed, jobs))


# ------------------------------------------------------------------------------------------ raw launches
def ag_gemm(slot, group, x_shard, a, b, out, M, N, K, a_mn, b_mn, epi, wait_mode, push=True, ack=True, gathered_b=False):
    """out (=|+=) op(A) op(B) where one operand is the gathered matrix staged in ``slot``."""
    if push:
        slot.epoch += 1
    tiles = ((M + BM - 1) // BM) * ((N + BN - 1) // BN)
    jobs = (group.nranks - 1) * slot.n_sub if slot.push_mode == 0 else slot.n_sub * slot.parts
    shard_bytes = slot.rows * slot.row_elems * 2
    send_bytes = shard_bytes if slot.push_mode == 2 else shard_bytes * (group.nranks - 1)
    n_comm = _comm_ctas(group.nranks, tiles, jobs, push, slot.push_mode, (M, N, K, send_bytes))
    gemm_ctas = min(_sms() - n_comm, tiles)
    rc = _lib.kernels().pd_ag_gemm(
        ptr(a), ptr(b), ptr(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)), c_int(b.stride(0)),
        c_int(out.stride(0)), c_int(a_mn), c_int(b_mn), c_int(epi), c_int(1 if gathered_b else 0), ptr(x_shard), c_int(slot.rows), c_int(SUB_ROWS),
        c_int(slot.row_elems), c_int(group.rank), c_int(group.nranks), c_int(n_comm), c_int(slot.epoch - slot.bias_host[0]),
        c_int(wait_mode), c_int(0 if push else 1), c_int(1 if ack else 0), slot.p_stage, slot.p_flags, slot.p_ack,
        ptr(slot.done), c_int(slot.done_base - slot.bias_host[1]), ptr(slot.bias), c_int(WAIT_MS),
        c_int(slot.push_mode), c_int(slot.parts), ctypes.c_ulonglong(slot.mc_stage if slot.push_mode == 2 else 0),
        ptr(_lib.status_buffer(out.device)), stream())
    check(rc, "pd_ag_gemm")
    if ack:
        slot.done_base += gemm_ctas
    native._count()
    return out


def _red_ctas(default, tiles, K, result_bytes):
    """Reducer CTAs of the in-switch reduce-scatter GEMM.  Every reducer is an SM the GEMM does not get, and 32 of them
    can cost the GEMM a whole extra wave (512 tiles: 4 waves on 128 SMs, 5 on 116); too few and the reduction of this
    rank's slab (one SM pulls ~13 GB/s of reduced rows) outlasts the GEMM.  Picks the count that minimises
    max(GEMM waves x tile time, reduction time + one tile).  ``PD_RS_RED_CTAS`` fixes it."""
    if "PD_RS_RED_CTAS" in os.environ:
        return default
    sms = _sms()
    tile_us = 2.0 * BM * BN * K / GEMM_FLOP_PER_US_PER_SM
    best, best_t = default, None
    for r in range(8, 49):
        gemm_us = -(-tiles // (sms - r)) * tile_us
        red_us = result_bytes / (r * PUSH_BYTES_PER_US_PER_CTA) + tile_us + 8.0
        t = max(gemm_us, red_us)
        if best_t is None or t < best_t - 0.5:
            best, best_t = r, t
    return best


def gemm_rs(slot, group, a, b, out, M, N, K, a_mn, b_mn):
    slot.epoch += 1
    if slot.mc:
        tiles = ((M + BM - 1) // BM) * ((N + BN - 1) // BN)
        n_red = _red_ctas(slot.n_red, tiles, K, slot.rows * N * 2)
        rc = _lib.kernels().pd_gemm_rs_mc(
            ptr(a), ptr(b), ptr(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)), c_int(b.stride(0)), c_int(a_mn),
            c_int(b_mn), c_int(slot.rows), c_int(group.rank), c_int(group.nranks), c_int(slot.epoch - slot.bias_host[0]),
            ptr(slot.block.local), ctypes.c_ulonglong(slot.mc_partial), slot.p_cnt, slot.p_ack, ptr(slot.done),
            ptr(slot.bias), c_int(n_red), c_int(WAIT_MS), ptr(_lib.status_buffer(out.device)), stream())
        check(rc, "pd_gemm_rs_mc")
        native._count()
        return out
    rc = _lib.kernels().pd_gemm_rs(
        ptr(a), ptr(b), ptr(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)), c_int(b.stride(0)), c_int(a_mn),
        c_int(b_mn), c_int(slot.rows), c_int(group.rank), c_int(group.nranks), c_int(slot.epoch - slot.bias_host[0]),
        slot.p_recv, slot.p_cnt, slot.p_ack, ptr(slot.done), ptr(slot.bias), c_int(WAIT_MS), ptr(_lib.status_buffer(out.device)), stream())
    check(rc, "pd_gemm_rs")
    native._count()
    return out


WGRAD_PLAIN = _env_int("PD_WGRAD_PLAIN", 1)


def ag_ack(slot, group):
    """Tell every rank that this rank is done with the matrix staged in ``slot`` for its current epoch."""
    rc = _lib.kernels().pd_ag_ack(c_int(group.rank), c_int(group.nranks), c_int(slot.epoch - slot.bias_host[0]),
                                  slot.p_ack, ptr(slot.done), ptr(slot.bias), stream())
    check(rc, "pd_ag_ack")
    slot.done_base += 1
    native._count()


def _wgrad(weight, a, b, M, N, K, slot, group, x_shard, push, ack, gathered_b=False):
    """dW (+)= A^T B with tokens as the reduction dimension; straight into main_grad when present.

    When nothing has to be pushed - the gathered operand is still staged from the forward (or the dgrad) launch - the
    product is an ordinary local GEMM over this GPU's own staging buffer, and the 2-CTA kernel runs it at twice the
    rate of the flag-driven one (143 vs 281 us for the 7B qkv shape on 2 GPUs); a one-thread launch then acknowledges
    the epoch to the peers."""
    mg = getattr(weight, "main_grad", None)
    if not push and WGRAD_PLAIN and native.GEMM_IMPL == "2cta":
        if slot.push_mode != 2:
            # the fused kernels read this rank's own rows straight from the shard, and only the multicast push writes
            # them into the staging buffer as well: complete the staged matrix first (a local copy of 1/n of it)
            r0 = group.rank * slot.rows
            slot.stage[r0:r0 + slot.rows].copy_(x_shard.detach().reshape(slot.rows, slot.row_elems))
        if mg is not None:
            native.gemm(a, b, trans_a=True, out=mg, accumulate=True)
        else:
            dw = native.gemm(a, b, trans_a=True)
        if ack:
            ag_ack(slot, group)
        if mg is not None:
            hook = getattr(weight, "_main_grad_ready_hook", None)
            if hook is not None:
                hook(weight)
            return None
        return dw
    if mg is not None:
        ag_gemm(slot, group, x_shard, a, b, mg, M, N, K, 1, 1, 2, 1, push, ack, gathered_b)
        hook = getattr(weight, "_main_grad_ready_hook", None)
        if hook is not None:
            hook(weight)
        return None
    dw = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    ag_gemm(slot, group, x_shard, a, b, dw, M, N, K, 1, 1, 0, 1, push, ack, gathered_b)
    return dw


# ------------------------------------------------------------------------------------------ autograd
class _AllGatherLinear(torch.autograd.Function):
    """y[T, out/n] = all_gather(x[T/n, in]) @ W[in, out/n]"""

    @staticmethod
    def forward(ctx, x, weight, group):
        x = x.contiguous()
        rows, K = x.shape
        n = group.nranks
        T, N = rows * n, weight.shape[1]
        keep = None
        if KEEP_GATHERED and ctx.needs_input_grad[1]:
            keep = _owned_slot(group, rows, K, weight)
        slot = keep if keep is not None else _slot("ag", group, rows, K)
        y = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
        # with an owned slot the acknowledgement is left to the weight-gradient GEMM of this layer's backward
        ag_gemm(slot, group, x, slot.stage, weight, y, T, N, K, 0, 1, 0, 0, push=True, ack=keep is None)
        if keep is not None:
            keep.pending_backward = True
        ctx.kept, ctx.kept_epoch = keep, (keep.epoch if keep is not None else 0)
        ctx.save_for_backward(x, weight)
        ctx.group, ctx.weight_ref = group, weight
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        group = ctx.group
        dy = dy.contiguous()
        rows, K = x.shape
        n = group.nranks
        T, N = rows * n, weight.shape[1]
        dx = dw = None
        if ctx.needs_input_grad[0]:
            rs = _slot("rs", group, rows, K)
            dx = torch.empty((rows, K), dtype=torch.bfloat16, device=x.device)
            gemm_rs(rs, group, dy, weight, dx, T, K, N, 0, 0)          # dX = dY W^T -> reduce-scatter
        kept = ctx.kept
        if kept is not None:
            if kept.epoch != ctx.kept_epoch:
                raise RuntimeError("the staged all-gather of this layer was overwritten before its backward ran")
            if ctx.needs_input_grad[1]:
                # x is still staged from forward: no second gather; this launch acknowledges the epoch
                dw = _wgrad(ctx.weight_ref, kept.stage, dy, K, N, T, kept, group, x, False, True)
            kept.pending_backward = False
        elif ctx.needs_input_grad[1]:
            slot = _slot("ag", group, rows, K)                          # re-gather x, overlapped with the dW GEMM
            dw = _wgrad(ctx.weight_ref, slot.stage, dy, K, N, T, slot, group, x, True, True)
        return dx, dw, None


class _LinearReduceScatter(torch.autograd.Function):
    """y[T/n, out] = reduce_scatter(x[T, in/n] @ W[in/n, out])"""

    @staticmethod
    def forward(ctx, x, weight, group):
        x = x.contiguous()
        T, K = x.shape
        n = group.nranks
        rows, N = T // n, weight.shape[1]
        slot = _slot("rs", group, rows, N)
        y = torch.empty((rows, N), dtype=torch.bfloat16, device=x.device)
        gemm_rs(slot, group, x, weight, y, T, N, K, 0, 1)
        ctx.save_for_backward(x, weight)
        ctx.group, ctx.weight_ref = group, weight
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        group = ctx.group
        dy = dy.contiguous()
        T, K = x.shape
        rows, N = dy.shape
        slot = _slot("ag", group, rows, N)
        dx = dw = None
        need_dw = ctx.needs_input_grad[1]
        if ctx.needs_input_grad[0]:
            dx = torch.empty((T, K), dtype=torch.bfloat16, device=x.device)
            # dX = all_gather(dY) W^T ; the gathered dY stays staged for the weight gradient
            ag_gemm(slot, group, dy, slot.stage, weight, dx, T, K, N, 0, 0, 0, 0, push=True, ack=not need_dw)
            if need_dw:
                dw = _wgrad(ctx.weight_ref, x, slot.stage, K, N, T, slot, group, dy, False, True, True)
        elif need_dw:
            dw = _wgrad(ctx.weight_ref, x, slot.stage, K, N, T, slot, group, dy, True, True, True)
        return dx, dw, None


class _LinearAllReduce(torch.autograd.Function):
    """y[T, out] = all_reduce(x[T, in/n] @ W[in/n, out]) for a row-parallel layer WITHOUT sequence parallelism
    (python/paddle/distributed/fleet/layers/mpu/mp_layers.py:715-732: matmul, then mp_allreduce).  Two-shot form: the
    GEMM -> reduce-scatter kernel leaves every rank with the reduced rows it owns (partial tiles travel from inside the
    GEMM's epilogue), and an all-gather of those slabs completes the all-reduce, so the reduction traffic overlaps the
    GEMM and only the gather - half of an all-reduce's bytes - runs behind it.  Backward needs no communication: dY is
    replicated, dX = dY W^T and dW = X^T dY are local GEMMs."""

    @staticmethod
    def forward(ctx, x, weight, group):
        x = x.contiguous()
        T, K = x.shape
        n = group.nranks
        rows, N = T // n, weight.shape[1]
        slot = _slot("rs", group, rows, N)
        y = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
        mine = y[group.rank * rows:(group.rank + 1) * rows]
        gemm_rs(slot, group, x, weight, mine, T, N, K, 0, 1)
        import torch.distributed as tdist
        tdist.all_gather_into_tensor(y, mine, group=group.process_group)
        ctx.save_for_backward(x, weight)
        ctx.weight_ref = weight
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = native.gemm(dy, weight, trans_b=True)
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.weight_ref, "main_grad", None)
            if mg is not None:
                native.gemm(x, dy, trans_a=True, out=mg, accumulate=True)
                hook = getattr(ctx.weight_ref, "_main_grad_ready_hook", None)
                if hook is not None:
                    hook(ctx.weight_ref)
            else:
                dw = native.gemm(x, dy, trans_a=True)
        return dx, dw, None


def linear_all_reduce_ok(x2d, weight, group):
    """Shapes the fused row-parallel all-reduce takes: bf16 on the GPU, tokens divisible into 128-row slabs per rank,
    16-byte rows."""
    return (x2d.is_cuda and x2d.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and group is not None
            and group.nranks in (2, 4, 8) and symm.supported() and x2d.shape[0] % (group.nranks * SUB_ROWS) == 0
            and x2d.shape[1] % 8 == 0 and weight.shape[1] % 8 == 0 and os.environ.get("PD_FUSED_ROW_AR", "1") != "0")


def linear_all_reduce(x, weight, group):
    return as_tensor(_LinearAllReduce.apply(x, weight, group))


def _shapes_ok(tokens_local_rows):
    return _ag_ok(tokens_local_rows)


def allgather_linear(x, weight, group):
    if x.shape[0] % SUB_ROWS != 0:
        raise ValueError(f"fused all-gather GEMM needs a multiple of {SUB_ROWS} tokens per rank, got {x.shape[0]}")
    return as_tensor(_AllGatherLinear.apply(x, weight, group))


def linear_reduce_scatter(x, weight, group):
    if (x.shape[0] // group.nranks) % SUB_ROWS != 0:
        raise ValueError(f"fused GEMM reduce-scatter needs a multiple of {SUB_ROWS} tokens per rank")
    return as_tensor(_LinearReduceScatter.apply(x, weight, group))
