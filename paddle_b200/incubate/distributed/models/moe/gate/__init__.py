"""Routers (python/paddle/incubate/distributed/models/moe/gate/: base_gate.py, naive_gate.py, gshard_gate.py,
switch_gate.py)."""
from __future__ import annotations

import math

import torch

from ......_core.tensor import as_tensor
from ......distributed import collective as C
from ......distributed.models.moe.utils import (_limit_by_capacity, _number_count, _prune_gate_by_capacity,
                                                  _random_routing)
from ...... import nn


class BaseGate(nn.Layer):
    def __init__(self, num_expert, world_size):
        super().__init__()
        self.world_size, self.num_expert = world_size, num_expert
        self.tot_expert = world_size * num_expert
        self.loss = None

    def forward(self, x):
        raise NotImplementedError("Please implement the forward function.")

    def set_loss(self, loss):
        self.loss = loss

    def get_loss(self, clear=True):
        loss = self.loss
        if clear:
            self.loss = None
        return loss


class NaiveGate(BaseGate):
    def __init__(self, d_model, num_expert, world_size, topk=2):
        super().__init__(num_expert, world_size)
        self.gate = nn.Linear(d_model, self.tot_expert)
        self.gate.weight.name = "gate_" + self.gate.weight.name
        self.gate.bias.name = "gate_" + self.gate.bias.name
        self.top_k = topk

    def forward(self, inp, return_all_scores=False):
        gate = self.gate(inp)
        val, idx = torch.topk(gate, k=self.top_k, dim=-1, largest=True, sorted=True)
        if return_all_scores:
            return as_tensor(val), as_tensor(idx), gate
        return as_tensor(val), as_tensor(idx)


def _capacity_limit(topk_idx, num_expert, world_size, capacity, group):
    """Per-expert capacity over the whole expert-parallel group (gate/utils.py ``limit_by_capacity``)."""
    with torch.no_grad():
        cap = torch.full((num_expert,), int(capacity), dtype=torch.int64, device=topk_idx.device)
        pos_count = _number_count(topk_idx, num_expert * world_size)
        if world_size > 1:
            glob = torch.empty_like(pos_count)
            C._alltoall_single_io(pos_count, glob, group=group)
        else:
            glob = pos_count
        # experts of this rank: counts arriving from every worker, clipped in worker order
        allowed = _limit_by_capacity(glob, cap, world_size)
        if world_size > 1:
            back = torch.empty_like(allowed)
            C._alltoall_single_io(allowed, back, group=group)
        else:
            back = allowed
        return _prune_gate_by_capacity(topk_idx, back, num_expert, world_size)


class GShardGate(NaiveGate):
    def __init__(self, d_model, num_expert, world_size, topk=2, capacity=(1.2, 2.4), random_routing=True, group=None):
        assert topk == 2, "topk should be 2 in gshard"
        super().__init__(d_model, num_expert, world_size)
        self.capacity, self.random_routing, self.group = capacity, random_routing, group

    def forward(self, x):
        topk_val, topk_idx, gate_score = super().forward(x, return_all_scores=True)
        s = gate_score.shape[0]
        top1 = topk_idx.reshape([-1, self.top_k])[:, 0]
        c_e = torch.bincount(top1, minlength=self.tot_expert).to(gate_score.dtype) / s
        m_e = torch.softmax(gate_score, dim=1).mean(0)
        self.set_loss(as_tensor(torch.mean(c_e * m_e) * (self.num_expert ** 2)))
        cap_rate = self.capacity[0 if self.training else 1]
        capacity = math.ceil(cap_rate * x.shape[0])
        topk_idx = _capacity_limit(topk_idx, self.num_expert, self.world_size, capacity, self.group)
        if self.random_routing:
            rand = torch.rand(gate_score.shape[0], device=x.device, dtype=torch.float32)
            topk_idx = _random_routing(topk_idx, topk_val.float(), rand)
        return topk_val, topk_idx


class SwitchGate(NaiveGate):
    def __init__(self, d_model, num_expert, world_size, topk=1, switch_eps=0.1, capacity=(1.2, 2.4), group=None):
        assert topk == 1, "topk should be 1 in switch"
        super().__init__(d_model, num_expert, world_size, topk=1)
        self.switch_eps, self.capacity, self.group = switch_eps, capacity, group

    def forward(self, inp):
        score = self.gate(inp)
        if self.training:
            noise = torch.rand_like(score) * 2 * self.switch_eps + 1.0 - self.switch_eps
            score = score * noise
        score = torch.softmax(score, dim=-1)
        top1_score, top1_idx = torch.topk(score, k=1, dim=-1, largest=True)
        cap_rate = self.capacity[0 if self.training else 1]
        capacity = math.ceil(cap_rate * inp.shape[0])
        top1_idx = _capacity_limit(as_tensor(top1_idx), self.num_expert, self.world_size, capacity, self.group)
        valid = top1_idx.reshape(-1)
        valid = valid[valid > -1]
        fraction = torch.bincount(valid, minlength=self.tot_expert).to(score.dtype) / max(valid.numel(), 1)
        prob = score.sum(0) / max(valid.numel(), 1)
        self.set_loss(as_tensor((fraction * prob).sum() * self.tot_expert))
        return as_tensor(top1_score), top1_idx
