"""``paddle.incubate`` operators: fused masked softmax, segment reductions, graph helpers
(python/paddle/incubate/operators/, python/paddle/incubate/tensor/math.py)."""
from __future__ import annotations

import torch

from .._core.tensor import as_tensor
from ..geometric import (reindex_graph as graph_reindex, sample_neighbors as graph_sample_neighbors,  # noqa: F401
                         segment_max, segment_mean, segment_min, segment_sum, send_u_recv)


def softmax_mask_fuse(x, mask, name=None):
    """softmax(x + mask) over the last axis (incubate/operators/softmax_mask_fuse.py)."""
    return as_tensor(torch.softmax(x.float() + mask.float(), -1).to(x.dtype))


def softmax_mask_fuse_upper_triangle(x):
    """Causal softmax: positions above the diagonal are masked."""
    S = x.shape[-1]
    m = torch.full((x.shape[-2], S), float("-inf"), device=x.device).triu(1)
    return as_tensor(torch.softmax(x.float() + m, -1).to(x.dtype))


def graph_send_recv(x, src_index, dst_index, pool_type="sum", out_size=None, name=None):
    return send_u_recv(x, src_index, dst_index, pool_type, out_size)


def graph_khop_sampler(row, colptr, input_nodes, sample_sizes, sorted_eids=None, return_eids=False, name=None):
    from ..geometric import reindex_graph, sample_neighbors
    nodes = input_nodes
    all_nb, all_cnt = [], []
    frontier = nodes
    for k in sample_sizes:
        nb, cnt = sample_neighbors(row, colptr, frontier, k)
        all_nb.append(nb), all_cnt.append(cnt)
        frontier = as_tensor(torch.unique(nb))
    src, dst, out = reindex_graph(nodes, all_nb[0], all_cnt[0])
    return src, dst, out, as_tensor(torch.arange(out.shape[0]))


def identity_loss(x, reduction="none"):
    if reduction in ("sum", 0):
        return x.sum()
    if reduction in ("mean", 1):
        return x.mean()
    return x
