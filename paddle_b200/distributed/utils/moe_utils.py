"""Expert-parallel token exchange (python/paddle/distributed/utils/moe_utils.py:31 ``global_scatter``, :154
``global_gather``; kernels paddle/phi/kernels/gpu/global_scatter_kernel.cu / global_gather_kernel.cu).

``local_count[i]`` = rows this rank sends to expert ``i`` (experts numbered rank-major: expert ``i`` lives on rank
``i // n_local_experts``); ``global_count[i]`` = rows this rank receives for its local expert ``i % n_local`` from
rank ``i // n_local``.  ``x`` is ordered by destination expert.  ``global_scatter`` returns the received rows ordered
by (local expert, source rank); ``global_gather`` is its inverse.  Both are differentiable (each is the other's
backward)."""
from __future__ import annotations

import torch

from ..._core.tensor import as_tensor
from .. import collective as C


def _nranks(group):
    if group is None and not C.is_initialized():
        return 1
    return C._grp(group).nranks


def _exchange(x, send_counts, recv_counts, group, n_local):
    """send_counts / recv_counts: python lists of length world * n_local (rank-major).  Returns rows received, laid
    out rank-major (source rank, local expert)."""
    n = _nranks(group)
    in_splits = [sum(send_counts[r * n_local:(r + 1) * n_local]) for r in range(n)]
    out_splits = [sum(recv_counts[r * n_local:(r + 1) * n_local]) for r in range(n)]
    out = torch.empty((sum(out_splits), *x.shape[1:]), dtype=x.dtype, device=x.device)
    if n == 1:
        out.copy_(x)
    else:
        C._alltoall_single_io(x.contiguous(), out, in_splits, out_splits, group=group)
    return C._plain(out)


def _rank_major_to_expert_major(rows, counts, n, n_local):
    """rows laid out (rank, expert) -> (expert, rank)."""
    if n_local == 1 or n == 1:
        return rows
    pieces = list(torch.split(rows, counts, 0))
    order = [r * n_local + e for e in range(n_local) for r in range(n)]
    return torch.cat([pieces[i] for i in order], 0)


def _expert_major_to_rank_major(rows, counts, n, n_local):
    if n_local == 1 or n == 1:
        return rows
    em_counts = [counts[r * n_local + e] for e in range(n_local) for r in range(n)]
    pieces = list(torch.split(rows, em_counts, 0))
    idx = {(e, r): i for i, (e, r) in enumerate((e, r) for e in range(n_local) for r in range(n))}
    return torch.cat([pieces[idx[(e, r)]] for r in range(n) for e in range(n_local)], 0)


class _GlobalScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, local_count, global_count, group):
        lc, gc = [int(v) for v in local_count.tolist()], [int(v) for v in global_count.tolist()]
        n = _nranks(group)
        n_local = len(lc) // n
        ctx.meta = (lc, gc, group, n, n_local)
        recv = _exchange(C._plain(x), lc, gc, group, n_local)
        return _rank_major_to_expert_major(recv, gc, n, n_local)

    @staticmethod
    def backward(ctx, g):
        lc, gc, group, n, n_local = ctx.meta
        rows = _expert_major_to_rank_major(g.contiguous(), gc, n, n_local)
        return _exchange(rows, gc, lc, group, n_local), None, None, None


class _GlobalGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, local_count, global_count, group):
        lc, gc = [int(v) for v in local_count.tolist()], [int(v) for v in global_count.tolist()]
        n = _nranks(group)
        n_local = len(lc) // n
        ctx.meta = (lc, gc, group, n, n_local)
        rows = _expert_major_to_rank_major(C._plain(x).contiguous(), gc, n, n_local)
        return _exchange(rows, gc, lc, group, n_local)

    @staticmethod
    def backward(ctx, g):
        lc, gc, group, n, n_local = ctx.meta
        recv = _exchange(g.contiguous(), lc, gc, group, n_local)
        return _rank_major_to_expert_major(recv, gc, n, n_local), None, None, None


def global_scatter(x, local_count, global_count, group=None, use_calc_stream=True):
    return as_tensor(_GlobalScatter.apply(x, local_count, global_count, group))


def global_gather(x, local_count, global_count, group=None, use_calc_stream=True):
    return as_tensor(_GlobalGather.apply(x, local_count, global_count, group))
