"""Mixtral-style sparse mixture-of-experts decoder: Llama attention (grouped-query), RMSNorm, rotary embedding, and in
every block a top-2 softmax router over SwiGLU experts with an auxiliary load-balancing loss.  Experts are spread
over an expert-parallel group (``moe_group``; each rank holds ``num_local_experts / group size`` of them) and tokens
travel through ``MoELayer``'s all-to-all dispatch / combine."""
from __future__ import annotations

import dataclasses

import torch

from .. import nn
from .._core.tensor import as_tensor
from ..incubate.distributed.models.moe import MoELayer
from ..incubate.distributed.models.moe.gate import NaiveGate
from ..nn.initializer import Normal
from ..ops import functional as K
from .llama import LlamaAttention, LlamaConfig, LlamaRMSNorm


@dataclasses.dataclass
class MixtralConfig(LlamaConfig):
    num_local_experts: int = 8
    num_experts_per_tok: int = 2
    router_aux_loss_coef: float = 0.02
    capacity_factor: float = 1.25
    expert_impl: str = "loop"           # "loop": one pair of Linear layers per expert; "grouped_fp8": stacked weights,
                                        # all local experts in one block-scaled fp8 grouped GEMM per projection

    @classmethod
    def mixtral_8x7b(cls, **kw):
        base = dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                    num_key_value_heads=8)
        base.update(kw)
        return cls(**base)

    @classmethod
    def tiny(cls, **kw):
        base = dict(vocab_size=512, hidden_size=256, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                    num_key_value_heads=1, num_local_experts=4, max_position_embeddings=256)
        base.update(kw)
        return cls(**base)


class MixtralExpert(nn.Layer):
    def __init__(self, config):
        super().__init__()
        init = nn.ParamAttr(initializer=Normal(0.0, config.initializer_range))
        self.gate_up_proj = nn.Linear(config.hidden_size, 2 * config.intermediate_size, weight_attr=init, bias_attr=False)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, weight_attr=init, bias_attr=False)

    def forward(self, x):
        return self.down_proj(K.swiglu(self.gate_up_proj(x)))


class SoftmaxTopKGate(NaiveGate):
    """Mixtral's router: softmax over all experts, top-k, re-normalised weights; auxiliary loss
    ``E * sum_e(fraction_e * mean_prob_e)``; tokens beyond ``capacity_factor * tokens * k / E`` per expert are dropped
    (index -1)."""

    def __init__(self, d_model, num_expert, world_size, topk=2, capacity_factor=1.25):
        super().__init__(d_model, num_expert, world_size, topk)
        self.capacity_factor = capacity_factor

    def forward(self, x):
        logits = self.gate(x).float()
        probs = torch.softmax(logits, -1)
        val, idx = torch.topk(probs, self.top_k, dim=-1)
        val = val / val.sum(-1, keepdim=True)
        E = self.tot_expert
        # one pass over a [T * k, E] one-hot gives the per-expert counts (no bincount: that one waits for the host)
        # and, through a running sum, each routed copy's arrival number at its expert
        flat = idx.reshape(-1)
        onehot = torch.nn.functional.one_hot(flat, E).to(torch.int32)
        frac = onehot.sum(0).to(probs.dtype) / flat.numel()
        self.set_loss(as_tensor(E * (frac * probs.mean(0)).sum()))
        if self.capacity_factor and self.capacity_factor > 0:
            cap = int(self.capacity_factor * x.shape[0] * self.top_k / E) + 1
            oh_t = onehot.t().contiguous()              # scan along the contiguous axis: [E, T * k]
            rank_in = ((oh_t.cumsum(1) - oh_t) * oh_t).sum(0)
            idx = torch.where(rank_in < cap, flat, torch.full_like(flat, -1)).reshape(idx.shape)
        return as_tensor(val.to(x.dtype)), as_tensor(idx)


class MixtralDecoderLayer(nn.Layer):
    def __init__(self, config, moe_group=None):
        super().__init__()
        self.input_layernorm = LlamaRMSNorm(config)
        self.self_attn = LlamaAttention(config)
        self.post_attention_layernorm = LlamaRMSNorm(config)
        world = moe_group.nranks if moe_group is not None else 1
        assert config.num_local_experts % world == 0
        n_local = config.num_local_experts // world
        gate = SoftmaxTopKGate(config.hidden_size, n_local, world, config.num_experts_per_tok, config.capacity_factor)
        if config.expert_impl == "grouped_fp8":
            from ..incubate.distributed.models.moe.fp8_experts import FP8GroupedExperts
            experts = FP8GroupedExperts(n_local, config.hidden_size, config.intermediate_size, config.initializer_range)
        else:
            experts = nn.LayerList([MixtralExpert(config) for _ in range(n_local)])
        self.moe = MoELayer(config.hidden_size, experts, gate=gate, moe_group=moe_group)

    def forward(self, hidden, residual, batch, seq):
        if residual is None:
            residual = hidden
            h = self.input_layernorm(hidden)
        else:
            h, residual = self.input_layernorm(hidden, residual)
        h = self.self_attn(h, batch, seq)
        h, residual = self.post_attention_layernorm(h, residual)
        return self.moe(h), residual


class MixtralForCausalLM(nn.Layer):
    def __init__(self, config: MixtralConfig, moe_group=None):
        super().__init__()
        self.config = config
        init = nn.ParamAttr(initializer=Normal(0.0, config.initializer_range))
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, weight_attr=init)
        self.layers = nn.LayerList([MixtralDecoderLayer(config, moe_group) for _ in range(config.num_hidden_layers)])
        self.norm = LlamaRMSNorm(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, weight_attr=init, bias_attr=False)
        if config.dtype != "float32":
            self.to(dtype=config.dtype)

    def forward(self, input_ids, labels=None):
        batch, seq = input_ids.shape
        h = self.embed_tokens(input_ids).reshape([batch * seq, self.config.hidden_size])
        residual, aux = None, 0.0
        for layer in self.layers:
            h, residual = layer(h, residual, batch, seq)
            aux = aux + layer.moe.gate.get_loss().float()
        h, _ = self.norm(h, residual)
        logits = self.lm_head(h)
        if labels is None:
            return logits.reshape([batch, seq, -1])
        loss = K.softmax_cross_entropy(logits, labels.reshape([-1])).mean()
        return loss + self.config.router_aux_loss_coef * aux
