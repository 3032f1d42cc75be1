"""Tensor-parallel glue operators (python/paddle/distributed/fleet/layers/mpu/mp_ops.py):
``_c_identity`` (identity fwd / all-reduce bwd, :41), ``_c_split`` (:57), ``_c_concat`` (all-gather on the
last axis), ``_mp_allreduce`` (all-reduce fwd / identity bwd, :226), ``_c_lookup_table`` (:310),
``_c_softmax_with_cross_entropy`` (:385), ``split`` (:773)."""
from __future__ import annotations

import torch

from ....._core.tensor import as_tensor
from .... import collective as C


def _plain(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


def _mp_group(group):
    if group is not None:
        return group
    from ... import fleet
    return fleet.get_hybrid_communicate_group().get_model_parallel_group()


class _CIdentity(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        C.all_reduce(dy, group=ctx.group)
        return dy, None


class _MpAllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        out = x.contiguous().clone()
        C.all_reduce(out, group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        return dy, None


class _CSplit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n, r = group.nranks, group.rank
        return x.chunk(n, -1)[r].contiguous()

    @staticmethod
    def backward(ctx, dy):
        g = ctx.group
        outs = []
        C.all_gather(outs, dy.contiguous(), g)
        return torch.cat(outs, -1), None


class _CConcat(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        outs = []
        C.all_gather(outs, x.contiguous(), group)
        return torch.cat(outs, -1)

    @staticmethod
    def backward(ctx, dy):
        g = ctx.group
        return dy.chunk(g.nranks, -1)[g.rank].contiguous(), None


def _c_identity(tensor, group=None, skip_c_identity_dynamic=False):
    g = _mp_group(group)
    if g is None or g.nranks == 1 or skip_c_identity_dynamic:
        return tensor
    return as_tensor(_CIdentity.apply(tensor, g))


def _mp_allreduce(tensor, op=C.ReduceOp.SUM, group=None, use_calc_stream=True, use_model_parallel=True,
                  skip_c_identity_dynamic=False):
    g = _mp_group(group)
    if g is None or g.nranks == 1:
        return tensor
    return as_tensor(_MpAllReduce.apply(tensor, g))


def _c_split(tensor, group=None):
    g = _mp_group(group)
    if g is None or g.nranks == 1:
        return tensor
    return as_tensor(_CSplit.apply(tensor, g))


def _c_concat(tensor, group=None):
    g = _mp_group(group)
    if g is None or g.nranks == 1:
        return tensor
    return as_tensor(_CConcat.apply(tensor, g))


def _c_lookup_table(table, index, start_index=0, vocab_size=-1, name=None):
    """Rows outside ``[start_index, start_index + rows)`` give zeros (c_embedding,
    paddle/phi/kernels/gpu/c_embedding_kernel.cu:31)."""
    from .....ops import functional as K
    return K.embedding(index, table, None, vocab_start=start_index, sharded=True)


class _EmbedExchange:
    """Symmetric-memory buffers of the fused vocab-parallel + sequence-sharded embedding for one group."""

    GRID = 128

    def __init__(self, group, shard_rows, row_bytes):
        import ctypes

        from .....parallel import symm
        self.n, self.rank = group.nranks, group.rank
        self.slot_bytes = (shard_rows * row_bytes + 255) // 256 * 256
        self.block = symm.SymmBlock(2 * self.slot_bytes + 256, group)
        u64x8 = ctypes.c_ulonglong * 8
        v = self.block.peer_ptrs(0)
        self.p_recv = u64x8(*(v + [0] * (8 - len(v))))
        v = self.block.peer_ptrs(2 * self.slot_bytes)
        self.p_cnt = u64x8(*(v + [0] * (8 - len(v))))
        self.seen = torch.zeros(2, dtype=torch.int32, device=self.block.local.device)


_embed_exchanges = {}


class _VocabEmbedToSeqShard(torch.autograd.Function):
    """ids [T] + weight shard [V / n, H] -> this rank's sequence shard [T / n, H] of the embedded tokens, in one kernel
    over peer memory (forward).  Backward gathers the shards' gradients (every rank needs the rows of its own
    vocabulary range from all tokens) and accumulates them into the weight shard's gradient."""

    @staticmethod
    def forward(ctx, ids, weight, group, vstart):
        from .....ops import _lib, native
        from .....ops._lib import c_int, c_int64, check, ptr, stream
        n = group.nranks
        ids = ids.reshape(-1).to(torch.int64).contiguous()
        T, H = ids.numel(), weight.shape[1]
        row_bytes = H * weight.element_size()
        key = id(group)
        ex = _embed_exchanges.get(key)
        if ex is None or ex.slot_bytes < (T // n) * row_bytes:
            ex = _embed_exchanges[key] = _EmbedExchange(group, T // n, row_bytes)
        out = torch.empty(T // n, H, dtype=weight.dtype, device=weight.device)
        w = weight.detach()
        rc = _lib.kernels().pd_embedding_scatter(
            ptr(ids), ptr(w), ptr(out), c_int64(T), c_int64(vstart), c_int64(w.shape[0]), c_int(row_bytes),
            c_int64(ex.slot_bytes), c_int(ex.rank), c_int(n), ex.p_recv, ex.p_cnt, ptr(ex.seen), c_int(min(ex.GRID, T)),
            c_int(2000), ptr(_lib.status_buffer(w.device)), stream())
        check(rc, "pd_embedding_scatter")
        native._count(2)
        ctx.save_for_backward(ids)
        ctx.group, ctx.vstart, ctx.wshape, ctx.wdtype = group, vstart, tuple(weight.shape), weight.dtype
        ctx.table_ref = weight
        return out

    @staticmethod
    def backward(ctx, g):
        (ids,) = ctx.saved_tensors
        n = ctx.group.nranks
        full = torch.empty(n * g.shape[0], g.shape[1], dtype=g.dtype, device=g.device)
        C.all_gather(full, g.contiguous(), group=ctx.group)
        from .....ops import native
        table = ctx.table_ref
        mg = getattr(table, "main_grad", None)
        if mg is not None:                       # fp32 accumulation buffer of the mixed-precision optimizers
            native.embedding_bwd(ids, _plain(full), mg, ctx.vstart, -1)
            hook = getattr(table, "_main_grad_ready_hook", None)
            if hook is not None:
                hook(table)
            return None, None, None, None
        dw = torch.zeros(ctx.wshape, dtype=torch.float32, device=g.device)
        native.embedding_bwd(ids, _plain(full), dw, ctx.vstart, -1)
        return None, dw.to(ctx.wdtype), None, None


def fused_embedding_available(weight, tokens, group):
    """The fused lookup needs a GPU with peer-mapped memory, 16-byte rows and a token count divisible by the group."""
    import os
    if os.environ.get("PD_FUSED_EMBEDDING", "1") == "0" or group is None or group.nranks == 1:
        return False
    from .....parallel import symm
    return (weight.is_cuda and symm.supported() and (weight.shape[1] * weight.element_size()) % 16 == 0
            and tokens % group.nranks == 0)


def vocab_parallel_embedding_to_sequence_shard(ids, weight, group, vocab_start):
    return as_tensor(_VocabEmbedToSeqShard.apply(_plain(ids), weight, group, int(vocab_start)))


class _CEExchange:
    """Symmetric-memory exchange buffers of the fused vocab-parallel cross entropy for one group: every rank's
    (max, sum-exp, target) triples land in every peer's buffer by plain stores and one kernel merges them."""

    def __init__(self, group, rows):
        import ctypes

        from .....parallel import symm
        self.n = group.nranks
        self.rank = group.rank
        self.rows_pad = (max(int(rows), 8192) + 255) // 256 * 256
        nblocks = self.rows_pad // 256
        recv = 2 * self.n * 3 * self.rows_pad * 4
        self.block = symm.SymmBlock(recv + nblocks * 4, group)
        u64x8 = ctypes.c_ulonglong * 8
        v = self.block.peer_ptrs(0)
        self.p_recv = u64x8(*(v + [0] * (8 - len(v))))
        v = self.block.peer_ptrs(recv)
        self.p_cnt = u64x8(*(v + [0] * (8 - len(v))))
        self.seen = torch.zeros(nblocks, dtype=torch.int32, device=self.block.local.device)

    def combine(self, mx, sm, tg, labels, ignore_index):
        from .....ops import _lib, native
        from .....ops._lib import c_int, c_int64, check, ptr, stream
        rows = mx.numel()
        lse, loss = torch.empty_like(mx), torch.empty_like(mx)
        labels = labels.reshape(-1).to(torch.int64)
        rc = _lib.kernels().pd_ce_combine(ptr(mx), ptr(sm), ptr(tg), ptr(labels), ptr(lse), ptr(loss), c_int64(rows),
                                          c_int64(self.rows_pad), c_int64(ignore_index), c_int(self.rank), c_int(self.n),
                                          self.p_recv, self.p_cnt, ptr(self.seen), c_int(2000),
                                          ptr(_lib.status_buffer(mx.device)), stream())
        check(rc, "pd_ce_combine")
        native._count()
        return lse, loss


_ce_exchanges = {}


def _ce_exchange(group, rows):
    """The group's exchange object, or None when symmetric memory is not available (CPU, ``PD_FUSED_CE=0``)."""
    import os
    if os.environ.get("PD_FUSED_CE", "1") == "0":
        return None
    from .....parallel import symm
    if not symm.supported():
        return None
    key = id(group)
    ex = _ce_exchanges.get(key)
    if ex is None or ex.rows_pad < rows:
        ex = _ce_exchanges[key] = _CEExchange(group, rows)
    return ex


class _ParallelCE(torch.autograd.Function):
    """Vocab-parallel softmax cross entropy.  Each rank computes (max, sum-exp, target logit) of its
    logits shard in one kernel pass; the three per-token fp32 vectors are combined across the group with
    one packed all-reduce pair (MAX then SUM) instead of the reference's three
    (c_softmax_with_cross_entropy_kernel.cu:229,309,322); backward writes (softmax - onehot) * dloss."""

    @staticmethod
    def forward(ctx, logits, labels, group, ignore_index):
        from .....ops import native
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V)
        if not l2.is_contiguous():
            l2 = l2.contiguous()
        lab = labels.reshape(-1)
        vstart = group.rank * V
        use_native = l2.is_cuda and l2.dtype in (torch.bfloat16, torch.float32) and V % 8 == 0
        if use_native:
            mx, sm, tg, _ = native.ce_stats(l2, lab, vstart, ignore_index, want_loss=False)
        else:
            lf = l2.float()
            mx = torch.amax(lf, -1)
            sm = torch.exp(lf - mx[:, None]).sum(-1)
            local = lab - vstart
            ok = (local >= 0) & (local < V) & (lab != ignore_index)
            tg = torch.where(ok, lf.gather(1, local.clamp(0, V - 1)[:, None]).squeeze(1), torch.zeros_like(mx))
        ex = _ce_exchange(group, l2.shape[0]) if use_native else None
        if ex is not None:
            lse, loss = ex.combine(mx, sm, tg, lab, ignore_index)
        else:
            gmx = mx.clone()
            C.all_reduce(gmx, C.ReduceOp.MAX, group)
            packed = torch.stack([sm * torch.exp(mx - gmx), tg])
            C.all_reduce(packed, C.ReduceOp.SUM, group)
            lse = gmx + packed[0].log()
            loss = torch.where(lab == ignore_index, torch.zeros_like(lse), lse - packed[1])
        ctx.save_for_backward(l2, lab, lse)
        ctx.vstart, ctx.ignore_index, ctx.use_native, ctx.shape = vstart, ignore_index, use_native, logits.shape
        return loss.view(labels.shape)

    @staticmethod
    def backward(ctx, dloss):
        from .....ops import native
        l2, lab, lse = ctx.saved_tensors
        dl = dloss.reshape(-1).contiguous().float()
        if ctx.use_native:
            d = native.ce_bwd(l2, lab, lse, dl, ctx.vstart, ctx.ignore_index)
        else:
            V = l2.shape[-1]
            p = torch.exp(l2.float() - lse[:, None])
            local = lab - ctx.vstart
            ok = (local >= 0) & (local < V)
            onehot = torch.zeros_like(p)
            onehot[ok, local[ok]] = 1.0
            d = ((p - onehot) * torch.where(lab == ctx.ignore_index, torch.zeros_like(dl), dl)[:, None]).to(l2.dtype)
        return d.view(ctx.shape), None, None, None


def _c_softmax_with_cross_entropy(logits, label, group=None, return_softmax=False, ignore_index=-100):
    g = _mp_group(group)
    lab = label.squeeze(-1) if label.dim() == logits.dim() else label
    if g is None or g.nranks == 1:
        from .....ops import functional as K
        loss = K.softmax_cross_entropy(logits, lab, ignore_index)
    else:
        loss = as_tensor(_ParallelCE.apply(logits, lab, g, ignore_index))
    loss = loss.unsqueeze(-1) if label.dim() == logits.dim() else loss
    if return_softmax:
        raise NotImplementedError("return_softmax is not supported for the vocab-parallel loss")
    return loss


def _c_softmax_with_multi_label_cross_entropy(logits, label, smooth_weight, group=None, return_softmax=False,
                                              ignore_index=-100, sum_multi_label_loss=True):
    """Vocab-parallel cross entropy against several labels per row, each weighted by ``smooth_weight``
    (mp_ops.py:461): ``loss[..., l] = smooth_weight[..., l] * CE(logits, label[..., l])``, summed over ``l`` when
    ``sum_multi_label_loss``.  ``label`` and ``smooth_weight`` are ``[..., L]``."""
    if label.shape != smooth_weight.shape:
        raise ValueError(f"label {list(label.shape)} and smooth_weight {list(smooth_weight.shape)} must agree")
    if label.dim() == logits.dim() - 1:
        label, smooth_weight = label.unsqueeze(-1), smooth_weight.unsqueeze(-1)
    losses = []
    for l in range(label.shape[-1]):
        one = _c_softmax_with_cross_entropy(logits, label[..., l], group=group, ignore_index=ignore_index)
        losses.append(one * smooth_weight[..., l].to(one.dtype))
    out = torch.stack(losses, -1)
    return as_tensor(out.sum(-1, keepdim=True) if sum_multi_label_loss else out)


def split(x, size, operation, axis=0, num_partitions=1, gather_out=True, weight_attr=None, bias_attr=None, name=None):
    """Build a parallel linear / embedding on the fly (mp_ops.py:773)."""
    from .mp_layers import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding
    if operation == "embedding":
        return VocabParallelEmbedding(size[0], size[1], weight_attr=weight_attr)(x)
    if operation == "linear":
        if axis == 0:
            return RowParallelLinear(size[0], size[1], weight_attr=weight_attr, has_bias=bias_attr is not False,
                                     input_is_parallel=False)(x)
        return ColumnParallelLinear(size[0], size[1], weight_attr=weight_attr, has_bias=bias_attr is not False,
                                    gather_output=gather_out)(x)
    raise ValueError(f"unknown operation {operation}")


# eager-mode names of the reference (mp_ops.py ``c_identity_eager`` ...): the autograd functions themselves
c_identity_eager = _CIdentity
mp_allreduce_eager = _MpAllReduce
c_split_eager = _CSplit
c_concat_eager = _CConcat
