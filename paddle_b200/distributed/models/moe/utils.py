"""Routing helpers (python/paddle/distributed/models/moe/utils.py: ``_number_count`` :25, ``_assign_pos`` :69,
``_random_routing`` :119, ``_limit_by_capacity`` :146, ``_prune_gate_by_capacity`` :191; kernels
paddle/phi/kernels/gpu/number_count_kernel.cu, assign_pos_kernel.cu, limit_by_capacity_kernel.cu,
prune_gate_by_capacity_kernel.cu, random_routing_kernel.cu)."""
from __future__ import annotations

import torch

from ...._core.tensor import as_tensor


def _number_count(numbers, upper_range):
    """How many entries of ``numbers`` equal each value in [0, upper_range); negative entries are ignored."""
    flat = numbers.reshape(-1)
    flat = flat[flat >= 0]
    return as_tensor(torch.bincount(flat, minlength=upper_range)[:upper_range].to(torch.int64))


def _assign_pos(x, cum_count):
    """Token indices grouped by expert: entry j of the result is the (flattened) index of the token routed to the
    expert whose cumulative range contains j.  Entries of ``x`` that are negative are dropped."""
    flat = x.reshape(-1)
    keep = torch.nonzero(flat >= 0).reshape(-1)
    order = torch.argsort(flat[keep], stable=True)
    return as_tensor(keep[order].to(torch.int64))


def _random_routing(topk_idx, topk_value, prob, topk=2):
    """GShard's random drop of the second expert: keep it only if ``2 * value > prob``."""
    if topk != 2:
        raise RuntimeError("only topk=2 is supported now")
    out = topk_idx.clone()
    drop = 2.0 * topk_value[:, 1] < prob
    out[:, 1] = torch.where(drop, torch.full_like(out[:, 1], -1), out[:, 1])
    return as_tensor(out)


def _limit_by_capacity(expert_count, capacity, n_worker):
    """Clip per-(worker, expert) counts so that each expert receives at most ``capacity[e]`` in worker order."""
    n_expert = capacity.numel()
    ec = expert_count.reshape(n_worker, n_expert).clone()
    left = capacity.clone().to(ec.dtype)
    for w in range(n_worker):
        take = torch.minimum(ec[w], left)
        ec[w] = take
        left = left - take
    return as_tensor(ec.reshape(-1))


def _prune_gate_by_capacity(gate_idx, expert_count, n_expert, n_worker):
    """Mark with -1 the tokens that exceed the (already limited) per-expert counts, first come first served."""
    flat = gate_idx.reshape(-1)
    out = flat.clone()
    limit = expert_count.reshape(-1).to(torch.int64)
    onehot = torch.nn.functional.one_hot(flat.clamp(min=0), n_expert * n_worker).to(torch.int64)
    onehot = onehot * (flat >= 0).unsqueeze(-1)
    # running count per expert: scanned along the contiguous axis of the transposed one-hot (a scan down the rows
    # of a [tokens, experts] matrix is ~70x slower on the GPU)
    oh_t = onehot.t().contiguous()
    rank_in_expert = ((oh_t.cumsum(1) - oh_t) * oh_t).sum(0)
    over = rank_in_expert >= limit[flat.clamp(min=0)]
    out[over | (flat < 0)] = -1
    return as_tensor(out.reshape(gate_idx.shape))
