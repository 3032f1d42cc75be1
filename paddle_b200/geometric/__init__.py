"""``paddle.geometric`` (python/paddle/geometric/): graph message passing (``send_u_recv``, ``send_ue_recv``,
``send_uv``), segment reductions, neighbour sampling and re-indexing."""
from __future__ import annotations

import torch

from .._core.tensor import as_tensor

__all__ = ["send_u_recv", "send_ue_recv", "send_uv", "segment_sum", "segment_mean", "segment_min", "segment_max",
           "reindex_graph", "reindex_heter_graph", "sample_neighbors", "weighted_sample_neighbors"]


def _p(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def _reduce(msg, index, n, op):
    index = _p(index).long()
    shape = (n, *msg.shape[1:])
    idx = index.reshape(-1, *([1] * (msg.dim() - 1))).expand_as(msg)
    if op == "sum":
        return torch.zeros(shape, dtype=msg.dtype, device=msg.device).scatter_add_(0, idx, msg)
    if op == "mean":
        s = torch.zeros(shape, dtype=msg.dtype, device=msg.device).scatter_add_(0, idx, msg)
        cnt = torch.bincount(index, minlength=n).clamp(min=1).reshape(-1, *([1] * (msg.dim() - 1)))
        return s / cnt.to(msg.dtype)
    red = "amax" if op == "max" else "amin"
    out = torch.zeros(shape, dtype=msg.dtype, device=msg.device)
    return out.scatter_reduce_(0, idx, msg, reduce=red, include_self=False)


def send_u_recv(x, src_index, dst_index, reduce_op="sum", out_size=None, name=None):
    x = _p(x)
    n = int(out_size) if out_size is not None else x.shape[0]
    return as_tensor(_reduce(x[_p(src_index).long()], dst_index, n, reduce_op))


def _combine(a, b, op):
    return {"add": a + b, "sub": a - b, "mul": a * b, "div": a / b}[op]


def send_ue_recv(x, y, src_index, dst_index, message_op="add", reduce_op="sum", out_size=None, name=None):
    x, y = _p(x), _p(y)
    gathered = x[_p(src_index).long()]
    if y.dim() < gathered.dim():                      # one value per edge: broadcast over the feature dims
        y = y.reshape(list(y.shape) + [1] * (gathered.dim() - y.dim()))
    msg = _combine(gathered, y, message_op)
    n = int(out_size) if out_size is not None else x.shape[0]
    return as_tensor(_reduce(msg, dst_index, n, reduce_op))


def send_uv(x, y, src_index, dst_index, message_op="add", name=None):
    return as_tensor(_combine(_p(x)[_p(src_index).long()], _p(y)[_p(dst_index).long()], message_op))


def _segment(data, ids, op):
    data, ids = _p(data), _p(ids).long()
    n = int(ids.max()) + 1 if ids.numel() else 0
    return as_tensor(_reduce(data, ids, n, op))


def segment_sum(data, segment_ids, name=None):
    return _segment(data, segment_ids, "sum")


def segment_mean(data, segment_ids, name=None):
    return _segment(data, segment_ids, "mean")


def segment_max(data, segment_ids, name=None):
    return _segment(data, segment_ids, "max")


def segment_min(data, segment_ids, name=None):
    return _segment(data, segment_ids, "min")


def reindex_graph(x, neighbors, count, value_buffer=None, index_buffer=None, name=None):
    """Relabel ``x`` (centre nodes) and their ``neighbors`` with consecutive ids; returns (reindex_src, reindex_dst,
    out_nodes)."""
    x, neighbors, count = _p(x).long(), _p(neighbors).long(), _p(count).long()
    nodes = torch.cat([x, neighbors])
    uniq, first = [], {}
    for v in nodes.tolist():
        if v not in first:
            first[v] = len(uniq)
            uniq.append(v)
    src = torch.tensor([first[v] for v in neighbors.tolist()], dtype=torch.int64)
    n = x.numel()
    if count.numel() != n and n and count.numel() % n == 0:
        # several edge types in one call: neighbours and counts of the types are concatenated
        dst = torch.cat([torch.repeat_interleave(torch.arange(n), count[i * n:(i + 1) * n]) for i in range(count.numel() // n)])
    else:
        dst = torch.repeat_interleave(torch.arange(n), count)
    return as_tensor(src), as_tensor(dst), as_tensor(torch.tensor(uniq, dtype=torch.int64))


def reindex_heter_graph(x, neighbors, count, value_buffer=None, index_buffer=None, name=None):
    """Several edge types over the same centre nodes ``x``: ``neighbors[i]`` / ``count[i]`` list the neighbours of each
    centre node under type i.  Ids are renumbered in one space: the centre nodes first, then every new neighbour in order
    of first appearance over the types.  -> (reindexed sources of all types concatenated, their destination = index
    of the centre node, the node list)."""
    centres = _p(x).long().tolist()
    ids = {v: i for i, v in enumerate(centres)}
    nodes = list(centres)
    src, dst = [], []
    for nb, c in zip(neighbors, count):
        for v in _p(nb).long().tolist():
            if v not in ids:
                ids[v] = len(nodes)
                nodes.append(v)
            src.append(ids[v])
        dst.append(torch.repeat_interleave(torch.arange(len(centres)), _p(c).long()))
    return (as_tensor(torch.tensor(src, dtype=torch.int64)), as_tensor(torch.cat(dst) if dst else torch.zeros(0, dtype=torch.int64)),
            as_tensor(torch.tensor(nodes, dtype=torch.int64)))


def sample_neighbors(row, colptr, input_nodes, sample_size=-1, eids=None, return_eids=False, perm_buffer=None, name=None):
    """CSC graph: neighbours of node v are ``row[colptr[v]:colptr[v+1]]``; up to ``sample_size`` of them per node."""
    row, colptr, nodes = _p(row).long(), _p(colptr).long(), _p(input_nodes).long()
    outs, counts, oe = [], [], []
    for v in nodes.tolist():
        lo, hi = int(colptr[v]), int(colptr[v + 1])
        idx = torch.arange(lo, hi)
        if 0 <= sample_size < idx.numel():
            idx = idx[torch.randperm(idx.numel())[:sample_size]]
        outs.append(row[idx])
        counts.append(idx.numel())
        if return_eids and eids is not None:
            oe.append(_p(eids)[idx])
    res = (as_tensor(torch.cat(outs) if outs else row[:0]), as_tensor(torch.tensor(counts, dtype=torch.int64)))
    return res + (as_tensor(torch.cat(oe)),) if return_eids and eids is not None else res


def weighted_sample_neighbors(row, colptr, edge_weight, input_nodes, sample_size=-1, eids=None, return_eids=False, name=None):
    row, colptr, nodes, w = _p(row).long(), _p(colptr).long(), _p(input_nodes).long(), _p(edge_weight).float()
    outs, counts = [], []
    for v in nodes.tolist():
        lo, hi = int(colptr[v]), int(colptr[v + 1])
        idx = torch.arange(lo, hi)
        if 0 <= sample_size < idx.numel():
            idx = idx[torch.multinomial(w[lo:hi], sample_size, replacement=False)]
        outs.append(row[idx])
        counts.append(idx.numel())
    return as_tensor(torch.cat(outs) if outs else row[:0]), as_tensor(torch.tensor(counts, dtype=torch.int64))
