"""Small GPT decoder (learned positions, LayerNorm, GELU FFN) built from the public ``nn`` layers; the
plumbing model of the CPU/gloo configuration and of the data-parallel / sharding parity tests."""
from __future__ import annotations

import dataclasses

import torch

from .. import nn
from ..nn import functional as F
from ..nn.initializer import Constant, Normal


@dataclasses.dataclass
class GPTConfig:
    vocab_size: int = 1024
    hidden_size: int = 128
    num_layers: int = 2
    num_heads: int = 4
    ffn_size: int = 512
    max_seq_len: int = 64
    initializer_range: float = 0.02
    dropout: float = 0.0


class GPTBlock(nn.Layer):
    def __init__(self, cfg):
        super().__init__()
        init = nn.ParamAttr(initializer=Normal(0.0, cfg.initializer_range))
        h = cfg.hidden_size
        self.ln1 = nn.LayerNorm(h)
        self.qkv = nn.Linear(h, 3 * h, weight_attr=init)
        self.proj = nn.Linear(h, h, weight_attr=init)
        self.ln2 = nn.LayerNorm(h)
        self.fc1 = nn.Linear(h, cfg.ffn_size, weight_attr=init)
        self.fc2 = nn.Linear(cfg.ffn_size, h, weight_attr=init)
        self.num_heads = cfg.num_heads

    def forward(self, x):
        b, s, h = x.shape
        qkv = self.qkv(self.ln1(x)).reshape([b, s, 3, self.num_heads, h // self.num_heads])
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.reshape([b, s, h]))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))


class GPTForCausalLM(nn.Layer):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.cfg = cfg
        init = nn.ParamAttr(initializer=Normal(0.0, cfg.initializer_range))
        self.wte = nn.Embedding(cfg.vocab_size, cfg.hidden_size, weight_attr=init)
        self.wpe = nn.Embedding(cfg.max_seq_len, cfg.hidden_size, weight_attr=init)
        self.blocks = nn.LayerList([GPTBlock(cfg) for _ in range(cfg.num_layers)])
        self.ln_f = nn.LayerNorm(cfg.hidden_size)
        self.head = nn.Linear(cfg.hidden_size, cfg.vocab_size, weight_attr=init, bias_attr=False)

    def forward(self, ids, labels=None):
        b, s = ids.shape
        pos = torch.arange(s, device=ids.device).unsqueeze(0)
        x = self.wte(ids) + self.wpe(pos)
        for blk in self.blocks:
            x = blk(x)
        logits = self.head(self.ln_f(x))
        if labels is None:
            return logits
        return F.cross_entropy(logits.reshape([-1, self.cfg.vocab_size]), labels.reshape([-1]))
