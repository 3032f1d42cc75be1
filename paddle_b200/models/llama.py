"""Llama-2 family decoder (RMSNorm, rotary embedding, SwiGLU, optional GQA) for training.

Built from this framework's public layers.  With ``tensor_parallel_degree > 1`` the projections become
``ColumnSequenceParallelLinear`` / ``RowSequenceParallelLinear`` over the fleet model-parallel group
and activations between blocks stay sharded on the sequence axis (Megatron sequence parallel, the
layout of python/paddle/distributed/fleet/utils/sequence_parallel_utils.py), the embedding and the
loss become vocab-parallel.  QKV and gate/up projections are fused into one GEMM each; residual adds
are fused into the following RMSNorm kernel.
"""
from __future__ import annotations

import dataclasses
import math

import torch

from .. import nn
from .._core.tensor import as_tensor
from ..nn import functional as F
from ..nn.initializer import Constant, Normal
from ..ops import functional as K


@dataclasses.dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int | None = None
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    initializer_range: float = 0.02
    tensor_parallel_degree: int = 1
    sequence_parallel: bool = True
    recompute: bool = False
    dtype: str = "bfloat16"
    fast_dispatch: bool = True

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads

    @property
    def head_dim(self):
        return self.hidden_size // self.num_attention_heads

    @classmethod
    def llama2_7b(cls, **kw):
        return cls(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32, **kw)

    @classmethod
    def llama2_13b(cls, **kw):
        return cls(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40, **kw)

    @classmethod
    def tiny(cls, **kw):
        base = dict(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                    num_attention_heads=2, max_position_embeddings=256)
        base.update(kw)
        return cls(**base)

    def num_params(self):
        h, f, v, L = self.hidden_size, self.intermediate_size, self.vocab_size, self.num_hidden_layers
        kv = self.num_key_value_heads * self.head_dim
        return 2 * v * h + L * (h * (h + 2 * kv) + h * h + 3 * h * f + 2 * h) + h

    def flops_per_token(self, seq_len):
        """Training FLOPs per token: 6 x matmul parameters plus causal attention."""
        h, L = self.hidden_size, self.num_hidden_layers
        dense = self.num_params() - self.vocab_size * h  # the embedding lookup does no matmul
        return 6 * dense + 6 * L * seq_len * h  # 12 L s h for full attention, halved by causality


def _linear_cls(config, kind):
    if config.tensor_parallel_degree <= 1:
        return None
    from ..distributed.fleet.layers.mpu import mp_layers
    from ..distributed.fleet.utils import sequence_parallel_utils as spu
    if config.sequence_parallel:
        return spu.ColumnSequenceParallelLinear if kind == "col" else spu.RowSequenceParallelLinear
    return mp_layers.ColumnParallelLinear if kind == "col" else mp_layers.RowParallelLinear


def _make_linear(config, in_f, out_f, kind):
    init = nn.ParamAttr(initializer=Normal(0.0, config.initializer_range))
    cls = _linear_cls(config, kind)
    if cls is None:
        return nn.Linear(in_f, out_f, weight_attr=init, bias_attr=False)
    if kind == "col":
        return cls(in_f, out_f, weight_attr=init, has_bias=False, gather_output=False)
    return cls(in_f, out_f, weight_attr=init, has_bias=False, input_is_parallel=True)


class LlamaRMSNorm(nn.Layer):
    def __init__(self, config):
        super().__init__()
        self.eps = config.rms_norm_eps
        self.weight = self.create_parameter([config.hidden_size], default_initializer=Constant(1.0))
        if config.tensor_parallel_degree > 1 and config.sequence_parallel:
            from ..distributed.fleet.utils.sequence_parallel_utils import mark_as_sequence_parallel_parameter
            mark_as_sequence_parallel_parameter(self.weight)

    def forward(self, x, residual=None):
        return K.rms_norm(x, self.weight, self.eps, residual)


class LlamaAttention(nn.Layer):
    def __init__(self, config):
        super().__init__()
        self.config = config
        tp = max(config.tensor_parallel_degree, 1)
        self.num_heads = config.num_attention_heads // tp
        self.num_kv_heads = max(config.num_key_value_heads // tp, 1)
        self.head_dim = config.head_dim
        q_out = config.num_attention_heads * self.head_dim
        kv_out = config.num_key_value_heads * self.head_dim
        self.qkv_proj = _make_linear(config, config.hidden_size, q_out + 2 * kv_out, "col")
        self.o_proj = _make_linear(config, q_out, config.hidden_size, "row")

    def forward(self, x, batch, seq):
        qkv = self.qkv_proj(x)                                   # [tokens, (hq + 2 hkv) * d] local heads
        d, hq, hkv = self.head_dim, self.num_heads, self.num_kv_heads
        if d == 128 and qkv.is_cuda and qkv.dtype == torch.bfloat16 and K.get_kernel_policy() == "fused" \
                and qkv.is_contiguous():
            # rope + attention directly on the packed projection (no slicing, one rope launch)
            from ..ops import attention
            cos, sin = K.rope_tables(seq, d, self.config.rope_theta, x.device, True)
            o = as_tensor(attention.rope_attention_packed(qkv, cos, sin, batch, seq, hq, hkv, True,
                                                          1.0 / math.sqrt(d)))
            return self.o_proj(o.reshape([-1, hq * d]))
        qkv = qkv.reshape([batch, seq, hq + 2 * hkv, d])
        q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
        cos, sin = K.rope_tables(seq, d, self.config.rope_theta, x.device, True)
        q, k = K.rope(q, cos, sin), K.rope(k, cos, sin)
        o = K.flash_attention(q, k, v, causal=True)              # [b, s, hq, d]
        return self.o_proj(o.reshape([-1, hq * d]))


class LlamaMLP(nn.Layer):
    def __init__(self, config):
        super().__init__()
        self.gate_up_proj = _make_linear(config, config.hidden_size, 2 * config.intermediate_size, "col")
        self.down_proj = _make_linear(config, config.intermediate_size, config.hidden_size, "row")

    def forward(self, x):
        return self.down_proj(K.swiglu(self.gate_up_proj(x)))


class LlamaDecoderLayer(nn.Layer):
    def __init__(self, config):
        super().__init__()
        self.input_layernorm = LlamaRMSNorm(config)
        self.self_attn = LlamaAttention(config)
        self.post_attention_layernorm = LlamaRMSNorm(config)
        self.mlp = LlamaMLP(config)

    def forward(self, hidden, residual, batch, seq):
        """``hidden`` is the previous block's branch output, ``residual`` the running stream; their sum
        is formed inside the norm kernel."""
        if residual is None:
            residual = hidden
            h = self.input_layernorm(hidden)
        else:
            h, residual = self.input_layernorm(hidden, residual)
        h = self.self_attn(h, batch, seq)
        h, residual = self.post_attention_layernorm(h, residual)
        h = self.mlp(h)
        return h, residual


class LlamaModel(nn.Layer):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        init = nn.ParamAttr(initializer=Normal(0.0, config.initializer_range))
        if config.tensor_parallel_degree > 1:
            from ..distributed.fleet.layers.mpu.mp_layers import VocabParallelEmbedding
            self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, weight_attr=init)
        else:
            self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, weight_attr=init)
        self.layers = nn.LayerList([LlamaDecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.norm = LlamaRMSNorm(config)

    def forward(self, input_ids):
        batch, seq = input_ids.shape
        sp = self.config.tensor_parallel_degree > 1 and self.config.sequence_parallel
        if sp:
            h = self.embed_tokens.forward_sequence_parallel(input_ids)
        else:
            h = self.embed_tokens(input_ids).reshape([batch * seq, self.config.hidden_size])
        residual = None
        for layer in self.layers:
            if self.config.recompute and self.training:
                from ..distributed.fleet.recompute import recompute
                h, residual = recompute(layer, h, residual, batch, seq)
            else:
                h, residual = layer(h, residual, batch, seq)
        h, _ = self.norm(h, residual)
        return h


class LlamaForCausalLM(nn.Layer):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        self.llama = LlamaModel(config)
        init = nn.ParamAttr(initializer=Normal(0.0, config.initializer_range))
        if config.tensor_parallel_degree > 1:
            from ..distributed.fleet.layers.mpu.mp_layers import ColumnParallelLinear, ParallelCrossEntropy
            from ..distributed.fleet.utils import sequence_parallel_utils as spu
            if config.sequence_parallel:
                self.lm_head = spu.ColumnSequenceParallelLinear(config.hidden_size, config.vocab_size, weight_attr=init,
                                                                has_bias=False, gather_output=False)
            else:
                self.lm_head = ColumnParallelLinear(config.hidden_size, config.vocab_size, weight_attr=init,
                                                    has_bias=False, gather_output=False)
            self.loss_fn = ParallelCrossEntropy()
        else:
            self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, weight_attr=init, bias_attr=False)
            self.loss_fn = None
        if config.dtype != "float32":
            self.to(dtype=config.dtype)

    def forward(self, input_ids, labels=None):
        """The stack runs with the Python-level tensor-subclass dispatch switched off: intermediate results are plain
        torch tensors (no per-operator ``__torch_function__`` round trip, which costs more host time than a small
        kernel takes on the GPU); only the returned value is wrapped again."""
        if not self.config.fast_dispatch:
            return self._forward(input_ids, labels)
        with torch._C.DisableTorchFunctionSubclass():
            out = self._forward(input_ids, labels)
        return as_tensor(out)

    def _forward(self, input_ids, labels=None):
        h = self.llama(input_ids)
        logits = self.lm_head(h)                                  # [tokens, vocab (/tp)]
        if labels is None:
            return logits.reshape([input_ids.shape[0], input_ids.shape[1], -1])
        flat = labels.reshape([-1])
        if self.loss_fn is not None:
            loss = self.loss_fn(logits, flat)
        else:
            loss = K.softmax_cross_entropy(logits, flat)
        return loss.mean()
