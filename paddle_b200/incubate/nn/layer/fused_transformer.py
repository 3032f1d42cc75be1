"""Fused transformer layers (python/paddle/incubate/nn/layer/fused_transformer.py: ``FusedMultiHeadAttention`` :196,
``FusedFeedForward`` :502, ``FusedTransformerEncoderLayer`` :737, ``FusedMultiTransformer`` :1071;
fused_linear.py, fused_dropout_add.py).

``FusedMultiTransformer`` keeps the reference's parameter layout (per-layer lists; qkv weight
``[3, num_heads, head_dim, embed_dim]`` when ``trans_qkvw``).  ``forward`` follows the reference semantics with dense
caches ``[2, B, H, max_seq, D]``.  For serving, ``prepare_paged()`` re-packs the weights once into GEMM-friendly
``[in, out]`` matrices and ``prefill_paged`` / ``decode_paged`` run the whole stack on this framework's kernels over a
paged KV cache: fused residual+RMSNorm, tcgen05 GEMMs (split-K for the skinny decode shapes), rotary + cache append,
flash attention for the prompt and the copy-engine-fed paged decode attention for generation; with ``nranks > 1``
the two row-parallel projections are followed by an all-reduce over the tensor-parallel group."""
from __future__ import annotations

import math

import torch

from ...._core.tensor import as_tensor
from ....nn import functional as F
from ....nn.initializer import Constant
from ....nn.layer.layers import Layer
from .. import functional as IF


class FusedLinear(Layer):
    def __init__(self, in_features, out_features, weight_attr=None, bias_attr=None, transpose_weight=False, name=None):
        super().__init__()
        shape = [out_features, in_features] if transpose_weight else [in_features, out_features]
        self.weight = self.create_parameter(shape, attr=weight_attr)
        self.bias = None if bias_attr is False else self.create_parameter([out_features], attr=bias_attr, is_bias=True)
        self.transpose_weight = transpose_weight

    def forward(self, x):
        return IF.fused_linear(x, self.weight, self.bias, self.transpose_weight)


class FusedDropoutAdd(Layer):
    def __init__(self, p=0.5, mode="upscale_in_train", name=None):
        super().__init__()
        self.p, self.mode = p, mode

    def forward(self, x, y):
        return IF.fused_dropout_add(x, y, self.p, self.training, self.mode)


class FusedDropout(Layer):
    """Dropout that may share one keep decision along some axes (python/paddle/incubate/nn/layer/fused_dropout_nd.py):
    with ``axis`` given the mask has size 1 on every other axis and is broadcast, so whole slices are dropped."""

    def __init__(self, p=0.5, axis=None, mode="upscale_in_train", name=None):
        super().__init__()
        if not isinstance(p, (float, int)) or p < 0 or p > 1:
            raise ValueError("p argument should be a number between 0 and 1")
        if mode not in ("downscale_in_infer", "upscale_in_train"):
            raise ValueError("mode argument should be 'downscale_in_infer' or 'upscale_in_train'")
        if axis is not None and not isinstance(axis, (int, list, tuple)):
            raise TypeError("datatype of axis argument should be int or list")
        self.p, self.axis, self.mode = float(p), axis, mode

    def forward(self, x):
        import torch
        if not self.training or self.p == 0.0:
            return x if self.mode == "upscale_in_train" or not self.training and self.p == 0 else x * (1.0 - self.p) \
                if self.mode == "downscale_in_infer" and not self.training else x
        if self.p == 1.0:
            return x * 0
        shape = list(x.shape)
        if self.axis is not None:
            axes = [self.axis] if isinstance(self.axis, int) else list(self.axis)
            shape = [s if i in [a % len(shape) for a in axes] else 1 for i, s in enumerate(shape)]
        keep = (torch.rand(shape, device=x.device) >= self.p).to(x.dtype)
        return x * keep / (1.0 - self.p) if self.mode == "upscale_in_train" else x * keep


class FusedBiasDropoutResidualLayerNorm(Layer):
    def __init__(self, embed_dim, dropout_rate=0.5, weight_attr=None, bias_attr=None, epsilon=1e-5, name=None):
        super().__init__()
        self.linear_bias = self.create_parameter([embed_dim], attr=bias_attr, is_bias=True)
        self.ln_scale = self.create_parameter([embed_dim], attr=weight_attr, default_initializer=Constant(1.0))
        self.ln_bias = self.create_parameter([embed_dim], attr=bias_attr, is_bias=True)
        self.dropout_rate, self.epsilon = dropout_rate, epsilon

    def forward(self, x, residual):
        return IF.fused_bias_dropout_residual_layer_norm(x, residual, self.linear_bias, self.ln_scale, self.ln_bias,
                                                         self.dropout_rate, self.epsilon, self.training)


class FusedMultiHeadAttention(Layer):
    def __init__(self, embed_dim, num_heads, dropout_rate=0.5, attn_dropout_rate=0.5, kdim=None, vdim=None,
                 normalize_before=False, need_weights=False, qkv_weight_attr=None, qkv_bias_attr=None,
                 linear_weight_attr=None, linear_bias_attr=None, pre_ln_scale_attr=None, pre_ln_bias_attr=None,
                 ln_scale_attr=None, ln_bias_attr=None, epsilon=1e-5, nranks=1, ring_id=-1, transpose_qkv_wb=False,
                 name=None):
        super().__init__()
        assert embed_dim % num_heads == 0
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads // nranks, embed_dim // num_heads
        self.normalize_before, self.ring_id, self.transpose_qkv_wb = normalize_before, ring_id, transpose_qkv_wb
        self.dropout_rate, self.attn_dropout_rate, self.epsilon = dropout_rate, attn_dropout_rate, epsilon
        nh, hd = self.num_heads, self.head_dim
        if transpose_qkv_wb:
            self.qkv_weight = self.create_parameter([embed_dim, 3 * nh * hd], attr=qkv_weight_attr)
            self.qkv_bias = self.create_parameter([3 * nh * hd], attr=qkv_bias_attr, is_bias=True)
        else:
            self.qkv_weight = self.create_parameter([3, nh, hd, embed_dim], attr=qkv_weight_attr)
            self.qkv_bias = self.create_parameter([3, nh, hd], attr=qkv_bias_attr, is_bias=True)
        self.linear_weight = self.create_parameter([nh * hd, embed_dim], attr=linear_weight_attr)
        self.linear_bias = self.create_parameter([embed_dim], attr=linear_bias_attr, is_bias=True)
        self.pre_ln_scale = self.create_parameter([embed_dim], attr=pre_ln_scale_attr, default_initializer=Constant(1.0))
        self.pre_ln_bias = self.create_parameter([embed_dim], attr=pre_ln_bias_attr, is_bias=True)
        self.ln_scale = self.create_parameter([embed_dim], attr=ln_scale_attr, default_initializer=Constant(1.0))
        self.ln_bias = self.create_parameter([embed_dim], attr=ln_bias_attr, is_bias=True)

    def forward(self, query, key=None, value=None, attn_mask=None, cache=None):
        return IF.fused_multi_head_attention(
            query, self.qkv_weight, self.linear_weight, self.normalize_before, self.pre_ln_scale, self.pre_ln_bias,
            self.ln_scale, self.ln_bias, self.epsilon, self.qkv_bias, self.linear_bias, cache, attn_mask,
            self.dropout_rate, self.attn_dropout_rate, self.epsilon, self.training, ring_id=self.ring_id,
            num_heads=self.num_heads, transpose_qkv_wb=self.transpose_qkv_wb)


class FusedFeedForward(Layer):
    def __init__(self, d_model, dim_feedforward, dropout_rate=0.1, epsilon=1e-5, activation="relu", act_dropout_rate=None,
                 normalize_before=False, linear1_weight_attr=None, linear1_bias_attr=None, linear2_weight_attr=None,
                 linear2_bias_attr=None, ln1_scale_attr=None, ln1_bias_attr=None, ln2_scale_attr=None,
                 ln2_bias_attr=None, nranks=1, ring_id=-1, name=None):
        super().__init__()
        ff = dim_feedforward // nranks
        self._linear1_weight = self.create_parameter([d_model, ff], attr=linear1_weight_attr)
        self._linear1_bias = self.create_parameter([ff], attr=linear1_bias_attr, is_bias=True)
        self._linear2_weight = self.create_parameter([ff, d_model], attr=linear2_weight_attr)
        self._linear2_bias = self.create_parameter([d_model], attr=linear2_bias_attr, is_bias=True)
        self._ln1_scale = self.create_parameter([d_model], attr=ln1_scale_attr, default_initializer=Constant(1.0))
        self._ln1_bias = self.create_parameter([d_model], attr=ln1_bias_attr, is_bias=True)
        self._ln2_scale = self.create_parameter([d_model], attr=ln2_scale_attr, default_initializer=Constant(1.0))
        self._ln2_bias = self.create_parameter([d_model], attr=ln2_bias_attr, is_bias=True)
        self._act, self._pre, self._eps, self._ring = activation, normalize_before, epsilon, ring_id
        self._p1 = dropout_rate if act_dropout_rate is None else act_dropout_rate
        self._p2 = dropout_rate

    def forward(self, src, cache=None):
        return IF.fused_feedforward(src, self._linear1_weight, self._linear2_weight, self._linear1_bias,
                                    self._linear2_bias, self._ln1_scale, self._ln1_bias, self._ln2_scale, self._ln2_bias,
                                    self._p1, self._p2, self._act, self._eps, self._eps, self._pre, self.training,
                                    ring_id=self._ring)


class FusedTransformerEncoderLayer(Layer):
    def __init__(self, d_model, nhead, dim_feedforward, dropout_rate=0.1, activation="relu", attn_dropout_rate=None,
                 act_dropout_rate=None, normalize_before=False, weight_attr=None, bias_attr=None):
        super().__init__()
        ad = dropout_rate if attn_dropout_rate is None else attn_dropout_rate
        self.fused_attn = FusedMultiHeadAttention(d_model, nhead, dropout_rate, ad, normalize_before=normalize_before)
        self.ffn = FusedFeedForward(d_model, dim_feedforward, dropout_rate, activation=activation,
                                    act_dropout_rate=act_dropout_rate, normalize_before=normalize_before)

    def forward(self, src, src_mask=None, cache=None):
        if cache is None:
            return self.ffn(self.fused_attn(src, attn_mask=src_mask))
        out, cache = self.fused_attn(src, attn_mask=src_mask, cache=cache)
        return self.ffn(out), cache


def _attr_list(attrs, i):
    if isinstance(attrs, (list, tuple)):
        return attrs[i]
    return attrs


class FusedMultiTransformer(Layer):
    def __init__(self, embed_dim, num_heads, dim_feedforward, dropout_rate=0.0, activation="gelu", normalize_before=True,
                 ln_scale_attrs=None, ln_bias_attrs=None, qkv_weight_attrs=None, qkv_bias_attrs=None,
                 linear_weight_attrs=None, linear_bias_attrs=None, ffn_ln_scale_attrs=None, ffn_ln_bias_attrs=None,
                 ffn1_weight_attrs=None, ffn1_bias_attrs=None, ffn2_weight_attrs=None, ffn2_bias_attrs=None,
                 epsilon=1e-5, residual_alpha=1.0, num_layers=-1, nranks=1, trans_qkvw=True, ring_id=-1,
                 norm_type="layernorm", use_neox_rotary_style=False, gqa_group_size=-1, name=None):
        super().__init__()
        assert embed_dim > 0 and num_heads > 0 and dim_feedforward > 0
        if num_layers < 0:
            assert isinstance(qkv_weight_attrs, (list, tuple))
            num_layers = len(qkv_weight_attrs)
        self.embed_dim, self.num_layers, self.nranks, self.ring_id = embed_dim, num_layers, nranks, ring_id
        self.head_dim = embed_dim // num_heads
        assert num_heads % nranks == 0 and dim_feedforward % nranks == 0
        self.num_heads = num_heads // nranks
        self.kv_heads = self.num_heads if gqa_group_size <= 0 else self.num_heads // gqa_group_size
        self.dim_ff = dim_feedforward // nranks
        self.activation, self.normalize_before, self.epsilon = activation, normalize_before, epsilon
        self.residual_alpha, self.trans_qkvw, self.norm_type = residual_alpha, trans_qkvw, norm_type
        self.use_neox_rotary_style, self.dropout_rate = use_neox_rotary_style, dropout_rate
        glu = activation in ("swiglu", "geglu")
        self.ln_scales, self.ln_biases, self.qkv_weights, self.qkv_biases = [], [], [], []
        self.linear_weights, self.linear_biases, self.ffn_ln_scales, self.ffn_ln_biases = [], [], [], []
        self.ffn1_weights, self.ffn1_biases, self.ffn2_weights, self.ffn2_biases = [], [], [], []
        nh, hd, E = self.num_heads, self.head_dim, embed_dim
        qkv_heads = nh + 2 * self.kv_heads

        def make(lst, key, shape, attrs, i, is_bias=False, init=None):
            attr = _attr_list(attrs, i)
            p = None if attr is False else self.create_parameter(shape, attr=attr, is_bias=is_bias, default_initializer=init)
            if p is not None:
                self.add_parameter(f"{key}_{i}", p)
            lst.append(p)
        for i in range(num_layers):
            make(self.ln_scales, "ln_scale", [E], ln_scale_attrs, i, init=Constant(1.0))
            make(self.ln_biases, "ln_bias", [E], ln_bias_attrs if norm_type == "layernorm" else False, i, True)
            qshape = ([3, nh, hd, E] if gqa_group_size <= 0 else [qkv_heads, hd, E]) if trans_qkvw else \
                ([E, 3, nh, hd] if gqa_group_size <= 0 else [E, qkv_heads, hd])
            make(self.qkv_weights, "qkv_weight", qshape, qkv_weight_attrs, i)
            make(self.qkv_biases, "qkv_bias", [qkv_heads * hd], qkv_bias_attrs, i, True)
            make(self.linear_weights, "linear_weight", [nh * hd, E], linear_weight_attrs, i)
            make(self.linear_biases, "linear_bias", [E], linear_bias_attrs, i, True)
            make(self.ffn_ln_scales, "ffn_ln_scale", [E], ffn_ln_scale_attrs, i, init=Constant(1.0))
            make(self.ffn_ln_biases, "ffn_ln_bias", [E], ffn_ln_bias_attrs if norm_type == "layernorm" else False, i, True)
            make(self.ffn1_weights, "ffn1_weight", [E, self.dim_ff * (2 if glu else 1)], ffn1_weight_attrs, i)
            make(self.ffn1_biases, "ffn1_bias", [self.dim_ff * (2 if glu else 1)], ffn1_bias_attrs, i, True)
            make(self.ffn2_weights, "ffn2_weight", [self.dim_ff, E], ffn2_weight_attrs, i)
            make(self.ffn2_biases, "ffn2_bias", [E], ffn2_bias_attrs, i, True)
        self._packed = None
        self._tp_group = None

    # ------------------------------------------------------------------ reference-semantics path (dense caches)
    def forward(self, src, attn_mask=None, caches=None, pre_caches=None, rotary_embs=None, rotary_emb_dims=0,
                beam_offset=None, seq_lens=None, time_step=None):
        if self.kv_heads != self.num_heads:
            raise NotImplementedError("dense-cache forward supports MHA; use the paged path for grouped-query attention")
        return IF.fused_multi_transformer(
            src, self.ln_scales, self.ln_biases, self.qkv_weights, self.qkv_biases, self.linear_weights,
            self.linear_biases, self.ffn_ln_scales, self.ffn_ln_biases, self.ffn1_weights, self.ffn1_biases,
            self.ffn2_weights, self.ffn2_biases, self.normalize_before, self.epsilon, self.residual_alpha, caches,
            beam_offset, pre_caches, seq_lens, rotary_embs, time_step, attn_mask, self.dropout_rate, rotary_emb_dims,
            self.activation, self.training, trans_qkvw=self.trans_qkvw, ring_id=self.ring_id, norm_type=self.norm_type,
            use_neox_rotary_style=self.use_neox_rotary_style)

    # ------------------------------------------------------------------ serving path (paged cache, native kernels)
    def prepare_paged(self, tp_group=None, max_batch=64):
        """Pack weights as ``[in, out]`` bf16 matrices and allocate the decode workspaces."""
        assert self.norm_type == "rmsnorm" and self.activation == "swiglu" and self.head_dim == 128, \
            "the paged path covers the Llama family: RMSNorm, SwiGLU, head_dim 128"
        E, nh, hkv, hd = self.embed_dim, self.num_heads, self.kv_heads, self.head_dim
        packed = []
        with torch.no_grad():
            for i in range(self.num_layers):
                w = self.qkv_weights[i]
                wq = (w.reshape([-1, E]).t() if self.trans_qkvw else w.reshape([E, -1])).contiguous()
                packed.append(dict(qkv=wq.detach(), out=self.linear_weights[i].detach(), ffn1=self.ffn1_weights[i].detach(),
                                   ffn2=self.ffn2_weights[i].detach(), ln=self.ln_scales[i].detach(),
                                   ffn_ln=self.ffn_ln_scales[i].detach(),
                                   qkv_b=None if self.qkv_biases[i] is None else self.qkv_biases[i].detach()))
        self._packed = packed
        self._tp_group = tp_group if (tp_group is not None and tp_group.nranks > 1) else None
        self._gar = None
        if self._tp_group is not None:
            from ....ops import functional as K
            from ....parallel import gemm_ar
            import os
            nccl_only = os.environ.get("PD_DECODE_NCCL_AR") == "1"     # baseline switch: GEMM + NCCL all-reduce
            if K.get_kernel_policy() == "fused" and not nccl_only and \
                    gemm_ar.supported(self._tp_group, E, min(max_batch, 128)):
                self._gar = gemm_ar.GemmAllReduce(self._tp_group, E, m_cap=min(max_batch, 128))
        dev = self.linear_weights[0].device
        from ....ops import native
        self._ws = {}
        for name, N, Kdim in (("qkv", (nh + 2 * hkv) * hd, E), ("out", E, nh * hd), ("ffn1", 2 * self.dim_ff, E),
                              ("ffn2", E, self.dim_ff)):
            s = native.suggest_splits(max_batch, N, Kdim) if dev.type == "cuda" else 1
            self._ws[name] = (s, torch.zeros((max_batch, N), dtype=torch.float32, device=dev) if s > 1 else None)
        return self

    def _gemm(self, name, x, w, residual=None):
        """x [M, K] @ w [K, N] (+ residual); split-K with fp32 reduce for the skinny decode shapes."""
        from ....ops import native
        M = x.shape[0]
        s, ws = self._ws[name]
        if s > 1 and M <= ws.shape[0]:
            acc = ws[:M]
            native.gemm_splitk(x, w, acc, s)
            return native.splitk_finalize(acc, residual=residual)
        y = native.gemm(x, w)
        if residual is not None:
            y = native.add_bf16(y, residual, out=y)
        return y

    def _all_reduce(self, t):
        if self._tp_group is not None:
            from ....distributed import collective as C
            C.all_reduce(t, group=self._tp_group)
        return t

    def _row_parallel(self, name, x, w, h_res):
        """Row-parallel projection + residual.  Returns (tensor, residual_included).  Single GPU: GEMM with the
        residual added in its epilogue pass.  Tensor parallel, decode-sized M: ONE kernel does the GEMM and the
        all-reduce over peer memory and adds the residual.  Otherwise: GEMM, NCCL all-reduce, residual added by the
        following norm kernel."""
        if self._tp_group is None:
            return self._gemm(name, x, w, residual=h_res), True
        if self._gar is not None and x.shape[0] <= self._gar.m_cap:
            return self._gar(x, w, residual=h_res), True
        o = self._gemm(name, x, w)
        self._all_reduce(o)
        return o, False

    def _mlp_and_out(self, i, h_res, attn_out2d):
        """Shared tail of a layer: out-projection + residual, RMSNorm, SwiGLU MLP; returns the tensor that the next
        layer's (residual+)RMSNorm consumes, the running residual, and whether that residual is still pending."""
        from ....ops import native
        P = self._packed[i]
        o, inc = self._row_parallel("out", attn_out2d, P["out"], h_res)
        if inc:
            h_res = o
            y, _, _ = native.rms_norm_fwd(o, P["ffn_ln"], self.epsilon)
        else:
            y, _, h_res = native.rms_norm_fwd(o, P["ffn_ln"], self.epsilon, residual=h_res, want_residual_out=True)
        g = self._gemm("ffn1", y, P["ffn1"])
        a = native.swiglu_fwd(g)
        f, inc = self._row_parallel("ffn2", a, P["ffn2"], h_res)
        return f, h_res, not inc

    def _layer_input(self, i, h, h_res, pending_tp):
        """RMSNorm of the layer input; under TP the previous layer's all-reduced MLP output is added to the residual
        inside the same kernel."""
        from ....ops import native
        P = self._packed[i]
        if pending_tp:
            y, _, h_res = native.rms_norm_fwd(h, P["ln"], self.epsilon, residual=h_res, want_residual_out=True)
            return y, h_res
        y, _, _ = native.rms_norm_fwd(h, P["ln"], self.epsilon)
        return y, h

    @torch.no_grad()
    def decode_paged(self, x, kv, cos64, sin64):
        """One token per sequence.  x [B, E] bf16; ``kv`` a PagedKVCache whose ``seq_lens`` hold the tokens already
        cached (the caller advances them after the step).  Returns [B, E]."""
        from ....ops import native
        B = x.shape[0]
        nh, hkv = self.num_heads, self.kv_heads
        h, h_res, pending = x, x, False
        q = torch.empty((B, nh, 128), dtype=x.dtype, device=x.device)
        nsplit = native.decode_attn_splits(B, hkv, kv.max_blocks_per_seq)
        wsp = None
        if nsplit > 1:
            wsp = (torch.empty((B, nh, nsplit, 128), dtype=torch.float32, device=x.device),
                   torch.empty((B, nh, nsplit, 2), dtype=torch.float32, device=x.device))
        scale = 1.0 / math.sqrt(128)
        for i in range(self.num_layers):
            P = self._packed[i]
            y, h_res = self._layer_input(i, h, h_res, pending)
            qkv = self._gemm("qkv", y, P["qkv"])
            native.decode_qkv_prep(qkv, P["qkv_b"], cos64, sin64, kv.seq_lens[:B], kv.block_table[:B], q, kv.k[i],
                                   kv.v[i], nh, hkv)
            o = native.paged_decode_attn(q, kv.k[i], kv.v[i], kv.block_table[:B], kv.seq_lens[:B], scale,
                                         nsplit=nsplit, len_offset=1, workspace=wsp)
            h, h_res, pending = self._mlp_and_out(i, h_res, o.view(B, nh * 128))
        if pending:
            h = native.add_bf16(h, h_res)
        return h

    @torch.no_grad()
    def prefill_paged(self, x, kv, cos, sin, batch, seq):
        """Prompt processing.  x [batch*seq, E] bf16 (all prompts have ``seq`` tokens); fills the caches at
        positions [0, seq) and returns [batch*seq, E]."""
        from ....ops import attention as A
        from ....ops import native
        nh, hkv = self.num_heads, self.kv_heads
        h, h_res, pending = x, x, False
        scale = 1.0 / math.sqrt(128)
        for i in range(self.num_layers):
            P = self._packed[i]
            y, h_res = self._layer_input(i, h, h_res, pending)
            qkv = native.gemm(y, P["qkv"])
            if P["qkv_b"] is not None:
                qkv += P["qkv_b"]
            o = A.rope_attention_packed(qkv, cos, sin, batch, seq, nh, hkv, True, scale)
            q4 = qkv.view(batch, seq, nh + 2 * hkv, 128)
            native.write_kv_cache(q4[:, :, nh:nh + hkv], q4[:, :, nh + hkv:], kv.block_table[:batch], kv.k[i], kv.v[i], 0)
            h, h_res, pending = self._mlp_and_out(i, h_res, o.reshape(batch * seq, nh * 128))
        if pending:
            h = native.add_bf16(h, h_res)
        return h
