"""Expert-parallel mixture-of-experts layer (python/paddle/incubate/distributed/models/moe/moe_layer.py:263
``MoELayer``; ``MoEScatter`` :99 / ``MoEGather`` :149; ``prepare_forward`` :226).

Flow per call: route (gate) -> count tokens per global expert and exchange the counts -> order the routed copies by
expert (``_assign_pos``) -> ``global_scatter`` (all-to-all with uneven splits) -> each local expert runs on its
contiguous slice -> ``global_gather`` -> copies return to their token/top-k slot and are combined with the gate
values.  Tokens pruned by the gate (index -1) contribute zeros."""
from __future__ import annotations

import torch

from ....._core.tensor import as_tensor
from ..... import nn
from .....distributed import collective as C
from .....distributed.models.moe.utils import _assign_pos, _number_count
from .....distributed.utils.moe_utils import global_gather, global_scatter
from .gate import BaseGate, GShardGate, NaiveGate, SwitchGate


def prepare_forward(gate, num_expert, world_size, moe_group):
    with torch.no_grad():
        local_expert_count = _number_count(gate, num_expert * world_size)
        if world_size > 1:
            global_expert_count = torch.empty_like(local_expert_count)
            C._alltoall_single_io(local_expert_count, global_expert_count, group=moe_group)
        else:
            global_expert_count = local_expert_count
        fwd_expert_count = global_expert_count.reshape(world_size, num_expert).sum(0)
        fwd_batch_size = int(fwd_expert_count.sum())
        pos = _assign_pos(gate, local_expert_count.cumsum(0))
    return pos, local_expert_count, as_tensor(global_expert_count), fwd_expert_count, fwd_batch_size


class MoELayer(nn.Layer):
    def __init__(self, d_model, experts, gate=None, moe_group=None, mp_group=None, recompute_interval=0,
                 recompute_ctx=None):
        super().__init__()
        self.recompute_interval = recompute_interval
        gate = gate if gate is not None else {}
        assert isinstance(gate, (dict, BaseGate)), "gate config' type must be dict or an instance of BaseGate"
        self.group = moe_group
        self.world_size = moe_group.nranks if moe_group is not None else 1
        self.num_expert = len(experts)
        self.d_model = d_model
        # either one layer per local expert, or one layer that holds all of them with stacked weights and runs them
        # as grouped GEMMs (``grouped = True``; ``forward(x, counts)``)
        self._grouped = bool(getattr(experts, "grouped", False))
        if self._grouped or isinstance(experts, nn.LayerList):
            self.experts = experts
        else:
            self.experts = nn.LayerList(list(experts))
        for p in self.experts.parameters():
            p.is_moe_param = True              # not synchronised by data parallelism: every rank owns other experts
            p.no_sync = True
        if isinstance(gate, dict):
            self.top_k = gate.get("top_k", 2)
            kind = gate.get("type", "gshard")
            if kind in ("naive", None):
                gate = NaiveGate(d_model, self.num_expert, self.world_size, topk=self.top_k)
            elif kind == "gshard":
                gate = GShardGate(d_model, self.num_expert, self.world_size, topk=self.top_k, group=self.group)
            elif kind == "switch":
                gate = SwitchGate(d_model, self.num_expert, self.world_size, topk=self.top_k, group=self.group)
            else:
                raise AssertionError(f"We only support naive gate, gshard gate and switch gate, but you choose {kind}")
        else:
            self.top_k = gate.top_k
        self.gate = gate

    # capacity of the fused exchange per (expert, source rank): ceil(factor * top_k * tokens / experts) rows, or
    # ``fused_capacity`` rows when set; routed copies beyond it are dropped (GShard capacity semantics)
    fused_capacity_factor = 1.25
    fused_capacity = None

    def _use_fused(self, inp):
        if not self._grouped or self.recompute_interval > 0 or self.world_size < 2:
            return False
        from .....parallel.moe_exchange import fused_moe_available
        return fused_moe_available(inp, self.experts, self.group)

    def _experts_forward(self, x, fwd_expert_count):
        if self._grouped:
            return self.experts(x, fwd_expert_count)
        outs, start = [], 0
        counts = [int(c) for c in fwd_expert_count.tolist()]
        for e, n in enumerate(counts):
            if n:
                outs.append(self.experts[e](x[start:start + n]))
            start += n
        return torch.cat(outs, 0) if outs else x.new_zeros((0, self.d_model))

    def forward(self, inp):
        origin_shape = inp.shape
        inp = inp.reshape([-1, origin_shape[-1]])
        value, gate = self.gate(inp)
        if self._use_fused(inp):
            # one autograd function: fp8-quantising dispatch over peer memory, grouped block-scaled GEMMs, weighted
            # combine; routing metadata stays on the device
            from .....parallel.moe_exchange import fused_moe_forward
            cap = self.fused_capacity
            cf = getattr(self.gate, "capacity_factor", None)
            if cap is None and cf:
                # a router that already prunes to a per-expert capacity over this rank's tokens: the receive regions are
                # sized to exactly that, so the exchange itself drops nothing
                k_ = gate.shape[1] if gate.dim() > 1 else 1
                cap = int(cf * inp.shape[0] * k_ / (self.num_expert * self.world_size)) + 1
            y = fused_moe_forward(C._plain(inp), C._plain(value), C._plain(gate), self.experts, self.group,
                                  capacity_factor=self.fused_capacity_factor, cap=cap)
            return as_tensor(y).reshape(origin_shape)
        pos, local_count, global_count, fwd_count, fwd_bs = prepare_forward(gate, self.num_expert, self.world_size,
                                                                            self.group)
        topk = gate.shape[1] if gate.dim() > 1 else 1
        token_of = pos // topk if topk > 1 else pos
        x = inp[token_of]                                                  # routed copies, ordered by expert
        x = global_scatter(x, local_count, global_count, self.group)
        if self.recompute_interval > 0 and x.requires_grad:
            from .....distributed.fleet.recompute import recompute
            x = recompute(self._experts_forward, x, fwd_count)
        else:
            x = self._experts_forward(x, fwd_count)
        x = global_gather(x, local_count, global_count, self.group)
        out = torch.zeros((inp.shape[0] * topk, self.d_model), dtype=x.dtype, device=x.device)
        out = out.index_copy(0, pos, C._plain(x))                           # dropped slots stay zero
        out = out.reshape(-1, topk, self.d_model)
        w = C._plain(value).reshape(out.shape[0], 1, topk).to(out.dtype)
        y = torch.bmm(w, out).reshape(-1, self.d_model)
        return as_tensor(y).reshape(origin_shape)
