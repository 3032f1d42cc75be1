"""Llama-family serving model: embedding + ``FusedMultiTransformer`` (paged KV cache) + final norm + lm head, with a
greedy generation loop.  The decode step is captured once into a CUDA graph (static shapes; sequence lengths and
block tables live in device memory that the graph reads), so generating a token costs one graph launch.

Tensor parallel: attention heads and the MLP inner dimension are split over the group (column-parallel qkv / ffn1,
row-parallel out / ffn2 followed by an all-reduce); the lm head is split over the vocabulary and the arg-max is
resolved from each rank's local (value, index) pair.  The reference builds the same computation from
``fused_multi_transformer`` (paddle/phi/kernels/fusion/gpu/fused_multi_transformer_kernel.cu:30) and leaves sampling
and the token loop to the serving library."""
from __future__ import annotations

import math

import torch

from .. import nn
from .._core.tensor import as_tensor
from ..incubate.nn import FusedMultiTransformer
from ..inference.paged_kv import PAGE, PagedKVCache
from ..nn.initializer import Normal
from ..ops import functional as K
from .llama import LlamaConfig


class LlamaForCausalLMInference(nn.Layer):
    def __init__(self, config: LlamaConfig, tp_group=None):
        super().__init__()
        self.config = config
        self.tp_group = tp_group if (tp_group is not None and tp_group.nranks > 1) else None
        n = self.tp_group.nranks if self.tp_group else 1
        self.nranks = n
        assert config.head_dim == 128 and config.num_attention_heads % n == 0 and config.vocab_size % n == 0
        init = nn.ParamAttr(initializer=Normal(0.0, config.initializer_range))
        gqa = config.num_attention_heads // config.num_key_value_heads
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, weight_attr=init)
        self.transformer = FusedMultiTransformer(
            config.hidden_size, config.num_attention_heads, config.intermediate_size, activation="swiglu",
            num_layers=config.num_hidden_layers, nranks=n, norm_type="rmsnorm", epsilon=config.rms_norm_eps,
            use_neox_rotary_style=True, qkv_weight_attrs=init, linear_weight_attrs=init, ffn1_weight_attrs=init,
            ffn2_weight_attrs=init, qkv_bias_attrs=False, linear_bias_attrs=False, ffn1_bias_attrs=False,
            ffn2_bias_attrs=False, gqa_group_size=gqa if gqa > 1 else -1, trans_qkvw=False)
        self.norm_weight = self.create_parameter([config.hidden_size], default_initializer=nn.initializer.Constant(1.0))
        self.lm_head = self.create_parameter([config.hidden_size, config.vocab_size // n], attr=init)
        self._graph = None
        self._kv = None
        if config.dtype != "float32":
            self.to(dtype=config.dtype)

    # ------------------------------------------------------------------ weights from a training model
    @torch.no_grad()
    def load_from_training(self, model, rank=0):
        """Copy (and, under tensor parallelism, slice) the weights of a ``LlamaForCausalLM`` built without TP."""
        n, r = self.nranks, rank
        cfg = self.config
        hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, 128
        self.embed_tokens.weight.copy_(model.llama.embed_tokens.weight)
        self.norm_weight.copy_(model.llama.norm.weight)
        self.lm_head.copy_(model.lm_head.weight.chunk(n, 1)[r])
        t = self.transformer
        for i, layer in enumerate(model.llama.layers):
            w = layer.self_attn.qkv_proj.weight                       # [E, (hq + 2 hkv) * d]
            q, k, v = w[:, :hq * d], w[:, hq * d:(hq + hkv) * d], w[:, (hq + hkv) * d:]
            loc = torch.cat([q.chunk(n, 1)[r], k.chunk(n, 1)[r], v.chunk(n, 1)[r]], 1)
            t.qkv_weights[i].copy_(loc.reshape(t.qkv_weights[i].shape))
            t.linear_weights[i].copy_(layer.self_attn.o_proj.weight.chunk(n, 0)[r])
            g, u = layer.mlp.gate_up_proj.weight.chunk(2, 1)
            t.ffn1_weights[i].copy_(torch.cat([g.chunk(n, 1)[r], u.chunk(n, 1)[r]], 1))
            t.ffn2_weights[i].copy_(layer.mlp.down_proj.weight.chunk(n, 0)[r])
            t.ln_scales[i].copy_(layer.input_layernorm.weight)
            t.ffn_ln_scales[i].copy_(layer.post_attention_layernorm.weight)
        return self

    # ------------------------------------------------------------------ engine
    def prepare(self, max_batch, max_seq_len, num_blocks=None):
        cfg = self.config
        dev = self.lm_head.device
        self.transformer.prepare_paged(self.tp_group, max_batch)
        if num_blocks is None:
            num_blocks = PagedKVCache.blocks_needed(max_batch, max_seq_len)
        self._kv = PagedKVCache(cfg.num_hidden_layers, self.transformer.kv_heads, num_blocks, max_batch, max_seq_len,
                                dtype=self.lm_head.dtype, device=dev)
        cos, sin = K.rope_tables(max_seq_len, 128, cfg.rope_theta, dev, True)
        self._cos, self._sin = cos, sin
        self._cos64, self._sin64 = cos[:, :64].contiguous(), sin[:, :64].contiguous()
        self._tokens = torch.zeros(max_batch, dtype=torch.int64, device=dev)
        self._graph, self._graph_batch = None, None
        return self

    def _logits(self, h):
        from ..ops import native
        y, _, _ = native.rms_norm_fwd(h, self.norm_weight.detach(), self.config.rms_norm_eps)
        return native.gemm(y, self.lm_head.detach())

    def _argmax(self, logits):
        """Greedy token from vocabulary-sharded logits."""
        val, idx = torch.max(logits.float(), -1)
        if self.tp_group is None:
            return idx
        from ..distributed import collective as C
        n, r = self.nranks, self.tp_group.rank
        idx = idx + r * (self.config.vocab_size // n)
        vals = torch.empty((n, *val.shape), dtype=val.dtype, device=val.device)
        idxs = torch.empty((n, *idx.shape), dtype=idx.dtype, device=idx.device)
        C.all_gather_into_tensor(vals, val.contiguous(), group=self.tp_group)
        C.all_gather_into_tensor(idxs, idx.contiguous(), group=self.tp_group)
        best = vals.argmax(0, keepdim=True)
        return idxs.gather(0, best)[0]

    def _pick(self, logits):
        """Next token per sequence: greedy, or one draw from the top-k / nucleus of softmax(logits / temperature)
        when sampling is configured (`generate(do_sample=True, ...)`).  Under tensor parallelism the vocabulary
        shards are gathered first; every rank draws with the same seed and counter, hence the same token."""
        cfg = getattr(self, "_sampling", None)
        if cfg is None:
            return self._argmax(logits)
        from ..ops import native
        if self.tp_group is not None:
            from ..distributed import collective as C
            parts = torch.empty((self.nranks, *logits.shape), dtype=logits.dtype, device=logits.device)
            C.all_gather_into_tensor(parts, logits.contiguous(), group=self.tp_group)
            logits = parts.permute(1, 0, 2).reshape(logits.shape[0], -1).contiguous()
        top_p, top_k, temperature, seed = cfg
        tp = self._top_p_buf[:logits.shape[0]]
        ids, _ = native.sample_top_p_top_k(logits, tp, top_k, temperature, seed, 0, draw_counter=self._draws)
        self._draws += 1                      # device-side: a replayed graph advances it as well
        return ids

    @torch.no_grad()
    def prefill(self, input_ids):
        """input_ids [B, S] (equal lengths).  Returns the first generated token per sequence [B]."""
        B, S = input_ids.shape
        kv = self._kv
        for b in range(B):
            assert kv.reserve(b, S), "KV cache pool exhausted"
        x = torch.nn.functional.embedding(input_ids.reshape(-1), self.embed_tokens.weight.detach())
        h = self.transformer.prefill_paged(x, kv, self._cos[:S].contiguous(), self._sin[:S].contiguous(), B, S)
        last = h.view(B, S, -1)[:, -1].contiguous()
        kv.seq_lens[:B] = S
        return self._pick(self._logits(last))

    def _decode_step(self, B):
        kv = self._kv
        x = torch.nn.functional.embedding(self._tokens[:B], self.embed_tokens.weight.detach())
        h = self.transformer.decode_paged(x, kv, self._cos64, self._sin64)
        nxt = self._pick(self._logits(h))
        self._tokens[:B].copy_(nxt)
        kv.seq_lens[:B] += 1

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens, use_cuda_graph=True, timings=None, do_sample=False, top_p=1.0,
                 top_k=0, temperature=1.0, seed=0):
        """Greedy decoding, or with ``do_sample`` top-k / nucleus sampling on the device (one sort-free kernel per
        step, Philox stream addressed by ``seed`` and a device-resident draw counter, so the captured decode step draws
        fresh numbers at every replay).  Returns int64 tokens [B, max_new_tokens]; ``timings`` (a dict) receives
        ``ttft_ms`` and ``decode_ms`` measured with CUDA events."""
        B, S = input_ids.shape
        sampling = (float(top_p), int(top_k), float(temperature), int(seed)) if do_sample else None
        if sampling != getattr(self, "_sampling", None):
            self._graph = None                # the captured step has the old choice baked in
        self._sampling = sampling
        if sampling is not None:
            dev = input_ids.device
            # the captured step holds on to these buffers: allocate once, reset in place
            if getattr(self, "_draws", None) is None:
                self._draws = torch.zeros(1, dtype=torch.int64, device=dev)
            else:
                self._draws.zero_()
            if getattr(self, "_top_p_buf", None) is None or self._top_p_buf.numel() < B:
                self._top_p_buf = torch.empty(max(B, 64), dtype=torch.float32, device=dev)
                self._graph = None
            self._top_p_buf.fill_(float(top_p))
        kv = self._kv
        kv.reset()
        for b in range(B):
            assert kv.reserve(b, S + max_new_tokens), "KV cache pool exhausted"
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if input_ids.is_cuda else None
        if ev:
            ev[0].record()
        first = self.prefill(input_ids)
        self._tokens[:B].copy_(first)
        out = torch.empty((B, max_new_tokens), dtype=torch.int64, device=input_ids.device)
        out[:, 0] = first
        if ev:
            ev[1].record()
        if use_cuda_graph and input_ids.is_cuda:
            if self._graph is None or self._graph_batch != B:
                # warm-up on a side stream (lazy initialisation), rewind the state, then capture
                lens0, tok0 = kv.seq_lens.clone(), self._tokens.clone()
                draws0 = self._draws.clone() if sampling is not None else None
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self._decode_step(B)
                torch.cuda.current_stream().wait_stream(side)
                kv.seq_lens.copy_(lens0), self._tokens.copy_(tok0)
                if draws0 is not None:
                    self._draws.copy_(draws0)             # the warm-up step drew once
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._decode_step(B)
                kv.seq_lens.copy_(lens0), self._tokens.copy_(tok0)
                self._graph, self._graph_batch = g, B
            if ev:
                ev[2].record()
            for t in range(1, max_new_tokens):
                self._graph.replay()
                out[:, t] = self._tokens[:B]
        else:
            if ev:
                ev[2].record()
            for t in range(1, max_new_tokens):
                self._decode_step(B)
                out[:, t] = self._tokens[:B]
        if ev:
            ev[3].record()
            torch.cuda.synchronize()
            if timings is not None:
                timings["ttft_ms"] = ev[0].elapsed_time(ev[1])
                timings["decode_ms"] = ev[2].elapsed_time(ev[3])
                timings["decode_tokens"] = B * (max_new_tokens - 1)
        return as_tensor(out)
