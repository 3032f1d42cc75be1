"""Parameter broadcast and fused gradient all-reduce helpers
(python/paddle/distributed/fleet/utils/hybrid_parallel_util.py:225-283)."""
from __future__ import annotations

import torch

from ... import collective as C


def _broadcast_params(model, group, src_rank, skip_distributed=False):
    if group is None or group.nranks == 1:
        return
    with torch.no_grad():
        for p in model.parameters():
            if skip_distributed and getattr(p, "is_distributed", False):
                continue
            C.broadcast(p.data, src_rank, group)
        for b in model.buffers():
            C.broadcast(b, src_rank, group)


def broadcast_mp_parameters(model, hcg):
    _broadcast_params(model, hcg.get_model_parallel_group(), hcg.get_model_parallel_group_src_rank(), True)


def broadcast_dp_parameters(model, hcg):
    _broadcast_params(model, hcg.get_data_parallel_group(), hcg.get_data_parallel_group_src_rank())


def broadcast_sharding_parameters(model, hcg):
    _broadcast_params(model, hcg.get_sharding_parallel_group(), hcg.get_sharding_parallel_group_src_rank())


def broadcast_sep_parameters(model, hcg):
    g = hcg.get_sep_parallel_group()
    if g is not None:
        _broadcast_params(model, g, g.ranks[0])


def broadcast_input_data(hcg, *inputs, **kwargs):
    g = hcg.get_model_parallel_group()
    if g is None or g.nranks == 1:
        return inputs, kwargs
    src = hcg.get_model_parallel_group_src_rank()
    for v in list(inputs) + list(kwargs.values()):
        if isinstance(v, torch.Tensor):
            with torch.no_grad():
                C.broadcast(v, src, g)
    return inputs, kwargs


def _grad_of(p):
    mg = getattr(p, "main_grad", None)
    return mg if mg is not None else torch.Tensor.grad.__get__(p)


def fused_allreduce_gradients_with_group(parameter_list, group, bucket_size=128 * 1024 * 1024, scale=None):
    """Flatten gradients into <= ``bucket_size`` byte buckets per dtype, all-reduce, scale, scatter back."""
    if group is None or group.nranks == 1:
        return
    grads = [g for g in (_grad_of(p) for p in parameter_list if p.requires_grad) if g is not None]
    buckets, cur, cur_bytes, cur_dtype = [], [], 0, None
    for g in grads:
        nb = g.numel() * g.element_size()
        if cur and (g.dtype != cur_dtype or cur_bytes + nb > bucket_size):
            buckets.append(cur)
            cur, cur_bytes = [], 0
        cur.append(g)
        cur_bytes += nb
        cur_dtype = g.dtype
    if cur:
        buckets.append(cur)
    scale = (1.0 / group.nranks) if scale is None else scale
    for b in buckets:
        flat = torch.cat([g.reshape(-1) for g in b]) if len(b) > 1 else b[0].reshape(-1)
        if scale != 1.0:
            flat.mul_(scale)
        C.all_reduce(flat, group=group)
        if len(b) > 1:
            off = 0
            for g in b:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()


def fused_allreduce_gradients(parameter_list, hcg):
    if hcg is None:
        return fused_allreduce_gradients_with_group(parameter_list, C._get_default_group())
    group = hcg.get_dp_sep_parallel_group() if hcg.get_sep_parallel_world_size() > 1 else hcg.get_data_parallel_group()
    fused_allreduce_gradients_with_group(parameter_list, group)


def sharding_reduce_gradients(parameter_list, hcg):
    g = hcg.get_sharding_parallel_group()
    fused_allreduce_gradients_with_group(parameter_list, g)


def obtain_optimizer_parameters_list(optimizer):
    """Flat parameter list of an optimizer, whether it was built from tensors or from parameter groups."""
    plist = getattr(optimizer, "_parameter_list", None) or []
    out = []
    for p in plist:
        if isinstance(p, dict):
            out.extend(p["params"])
        else:
            out.append(p)
    return out


def unwrap_optimizer(optimizer, optimizer_instances=()):
    """Peels wrapper optimizers (``_inner_opt`` / ``_optim`` / ``_optimizer``) until an instance of
    ``optimizer_instances`` (or the innermost optimizer) is reached."""
    cur = optimizer
    while True:
        if optimizer_instances and isinstance(cur, tuple(optimizer_instances)):
            return cur
        nxt = None
        for attr in ("_inner_opt", "_optim", "_optimizer", "_inner_optimizer"):
            nxt = cur.__dict__.get(attr) if hasattr(cur, "__dict__") else None
            if nxt is not None:
                break
        if nxt is None:
            return cur
        cur = nxt
