"""Helpers of the sharded checkpoint (python/paddle/distributed/checkpoint/utils.py: ``compute_local_shape_and_
global_offset`` :52, ``flatten_state_dict`` :77)."""
from __future__ import annotations

import torch

from ..auto_parallel.dist_tensor import is_dist
from .. import collective as C


def compute_local_shape_and_global_offset(global_shape, mesh, placements):
    coord = mesh.coord_of(C.get_rank())
    if coord is None:
        return None, None
    shape, offset = list(global_shape), [0] * len(global_shape)
    for a, p in enumerate(placements):
        if p.is_shard():
            n = mesh.shape[a]
            assert shape[p.dim] % n == 0
            shape[p.dim] //= n
            offset[p.dim] += coord[a] * shape[p.dim]
    return tuple(shape), tuple(offset)


def flatten_state_dict(sd, prefix=(), out=None, mapping=None):
    """Nested dicts -> one level keyed by dotted paths; returns (flat, {flat_key: path tuple})."""
    out = {} if out is None else out
    mapping = {} if mapping is None else mapping
    for k, v in sd.items():
        path = (*prefix, k)
        if isinstance(v, dict):
            flatten_state_dict(v, path, out, mapping)
        else:
            key = ".".join(str(p) for p in path)
            out[key], mapping[key] = v, path
    return out, mapping


def unflatten_state_dict(flat, mapping):
    out = {}
    for key, v in flat.items():
        path = mapping.get(key, (key,))
        d = out
        for p in path[:-1]:
            d = d.setdefault(p, {})
        d[path[-1]] = v
    return out


def describe(t):
    """(local tensor, global shape, local shape, global offset, replica_id) of a state-dict value; replica_id 0
    marks the copy that gets written when several ranks hold the same shard."""
    if is_dist(t):
        mesh, pl = t.process_mesh, t.placements
        shape, off = compute_local_shape_and_global_offset(t.shape, mesh, pl)
        if shape is None:
            return None
        coord = mesh.coord_of(C.get_rank())
        replica = sum(coord[a] for a, p in enumerate(pl) if not p.is_shard())
        from ..auto_parallel.dist_tensor import local_of
        return local_of(t).detach(), tuple(t.shape), shape, off, replica
    if isinstance(t, torch.Tensor):
        return t.detach().as_subclass(torch.Tensor), tuple(t.shape), tuple(t.shape), (0,) * t.dim(), C.get_rank()
    return None
