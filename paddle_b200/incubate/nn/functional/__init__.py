"""``paddle.incubate.nn.functional`` fused operators (python/paddle/incubate/nn/functional/*.py).

On a GPU with bf16 inputs the hot ones run this framework's kernels (rms_norm with fused residual, rotary
embedding, swiglu, the tcgen05 GEMM, paged decode attention); everything else, and every CPU call, is expressed
with plain tensor operators so that semantics can be checked anywhere."""
from __future__ import annotations

import math

import torch

from ...._core.tensor import as_tensor
from ....nn import functional as F
from ....ops import functional as K

__all__ = [
    "fused_multi_head_attention", "fused_feedforward", "fused_multi_transformer", "fused_matmul_bias", "fused_linear",
    "fused_linear_activation", "fused_bias_dropout_residual_layer_norm", "fused_moe", "moe_dispatch", "moe_ffn",
    "moe_reduce", "fused_dropout_add", "fused_rotary_position_embedding", "variable_length_memory_efficient_attention",
    "fused_rms_norm", "fused_layer_norm", "fused_bias_act", "masked_multihead_attention", "blha_get_max_len",
    "block_multihead_attention", "swiglu",
]


def _act(name):
    return {"gelu": F.gelu, "relu": F.relu, "silu": F.silu, "swish": F.silu, "none": lambda x: x, None: lambda x: x,
            "geglu": lambda x: F.gelu(x.chunk(2, -1)[0]) * x.chunk(2, -1)[1], "swiglu": swiglu}[name]


def swiglu(x, y=None, name=None):
    """``silu(x) * y``; with ``y=None`` the last axis of ``x`` is split in two halves (swiglu.py:24)."""
    return K.swiglu(x, y)


def fused_rms_norm(x, norm_weight, norm_bias, epsilon, begin_norm_axis, bias=None, residual=None, quant_scale=-1,
                   quant_round_type=0, quant_max_bound=0, quant_min_bound=0):
    """Returns ``(out, residual_out)`` when ``residual`` is given, else ``out`` (fused_rms_norm.py:59):
    ``residual_out = x + bias + residual``, ``out = rms_norm(residual_out) * weight + norm_bias``."""
    if quant_scale > 0:
        raise NotImplementedError("int8 output quantisation of fused_rms_norm is not provided")
    shape = x.shape
    lead = int(math.prod(shape[:begin_norm_axis]))
    x2 = x.reshape([lead, -1])
    if bias is not None:
        x2 = x2 + bias
    if residual is not None:
        out, res = K.rms_norm(x2, norm_weight, epsilon, residual=residual.reshape([lead, -1]))
    else:
        out, res = K.rms_norm(x2, norm_weight, epsilon), None
    if norm_bias is not None:
        out = out + norm_bias
    out = out.reshape(shape)
    return (out, res.reshape(shape)) if residual is not None else out


def fused_layer_norm(x, norm_weight, norm_bias, epsilon, residual_alpha=1.0, begin_norm_axis=1, bias=None,
                     residual=None, quant_scale=-1, quant_round_type=0, quant_max_bound=0, quant_min_bound=0):
    shape = x.shape
    lead = int(math.prod(shape[:begin_norm_axis]))
    x2 = x.reshape([lead, -1])
    if bias is not None:
        x2 = x2 + bias
    res = None
    if residual is not None:
        x2 = x2 + residual_alpha * residual.reshape([lead, -1])
        res = x2
    if norm_weight is None and norm_bias is None:
        out = x2
    else:
        out = K.layer_norm(x2, x2.shape[-1], norm_weight, norm_bias, epsilon)
    out = out.reshape(shape)
    return (out, res.reshape(shape)) if residual is not None else out


def fused_rotary_position_embedding(q, k=None, v=None, sin=None, cos=None, position_ids=None,
                                    use_neox_rotary_style=True, time_major=False, rotary_emb_base=10000.0):
    """q/k/v: ``[batch, seq, heads, head_dim]``.  ``use_neox_rotary_style=True`` rotates adjacent pairs
    (the reference's naming, fused_rope_utils.h:236), ``False`` rotates the two halves."""
    if time_major:
        q, k, v = (t.transpose([1, 0, 2, 3]) if t is not None else None for t in (q, k, v))
    seq, dim = q.shape[1], q.shape[-1]
    half_style = not use_neox_rotary_style
    if cos is None or sin is None:
        n = seq if position_ids is None else int(as_tensor(position_ids).max()) + 1
        cos_t, sin_t = K.rope_tables(max(n, seq), dim, rotary_emb_base, q.device, half_style)
    else:
        cos_t, sin_t = cos.reshape([-1, dim]).float(), sin.reshape([-1, dim]).float()
    outs = tuple(K.rope(t, cos_t, sin_t, position_ids=position_ids, half_style=half_style) if t is not None else None
                 for t in (q, k))
    outs = outs + (v,)
    if time_major:
        outs = tuple(t.transpose([1, 0, 2, 3]) if t is not None else None for t in outs)
    return outs


def fused_matmul_bias(x, y, bias=None, transpose_x=False, transpose_y=False, name=None):
    if transpose_x:
        x = x.transpose(-1, -2) if isinstance(x, torch.Tensor) else x
    w = y.t() if transpose_y else y
    return F.linear(x, w, bias)


def fused_linear(x, weight, bias=None, transpose_weight=False, name=None):
    return fused_matmul_bias(x, weight, bias, False, transpose_weight)


def _kernel_ok(t):
    return isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.bfloat16 and K._POLICY == "fused"


def fused_linear_activation(x, y, bias, trans_x=False, trans_y=False, activation=None):
    """``act(x @ y + bias)`` (fused_matmul_bias.py:113; kernel paddle/phi/kernels/fusion/gpu/fused_gemm_epilogue_kernel.cu).
    Without autograd the bias and the activation run in the GEMM epilogue; under autograd the pre-activation is needed
    for the backward pass, so only the bias is fused."""
    from ....ops import native
    act = activation if activation not in ("", "none") else None
    needs_grad = torch.is_grad_enabled() and any(isinstance(t, torch.Tensor) and t.requires_grad for t in (x, y, bias))
    if (not needs_grad and _kernel_ok(x) and _kernel_ok(y) and y.dim() == 2 and act in native.ACT_CODES and not trans_x
            and x.shape[-1] % 8 == 0 and y.shape[0] % 8 == 0 and y.shape[1] % 8 == 0 and y.is_contiguous()
            and (bias is None or (_kernel_ok(bias) and bias.is_contiguous()))):
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        out = native.gemm_epilogue(x2, y, bias, act, trans_b=bool(trans_y))
        return as_tensor(out.view(*x.shape[:-1], out.shape[-1]))
    return _act(activation)(fused_matmul_bias(x, y, bias, trans_x, trans_y))


def fused_linear_swiglu_interleaved(x, weight_interleaved):
    """First feed-forward GEMM with its activation: ``weight_interleaved [in, 2F]`` holds the gate and up projections
    with their columns interleaved (gate_0, up_0, gate_1, up_1, ...: see :func:`interleave_gate_up`); returns
    ``silu(x @ gate) * (x @ up)`` as ``[..., F]`` from one kernel - the ``[..., 2F]`` product never reaches memory.
    Inference path (no autograd: the backward pass would need the product)."""
    from ....ops import native
    x2 = x.reshape(-1, x.shape[-1])
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    if _kernel_ok(x2) and _kernel_ok(weight_interleaved) and weight_interleaved.shape[1] % 16 == 0:
        out = native.gemm_epilogue(x2, weight_interleaved, swiglu=True)
    else:
        h = torch.matmul(x2, weight_interleaved)
        out = torch.nn.functional.silu(h[:, 0::2]) * h[:, 1::2]
    return as_tensor(out.view(*x.shape[:-1], out.shape[-1]))


def interleave_gate_up(gate_weight, up_weight):
    """``[in, F]`` gate and up projection weights as one ``[in, 2F]`` matrix with interleaved columns."""
    return torch.stack([gate_weight, up_weight], -1).reshape(gate_weight.shape[0], -1).contiguous()


def fused_bias_act(x, bias=None, dequant_scales=None, shift=None, smooth=None, act_method="gelu",
                   compute_dtype="default", quant_scale=-1, quant_round_type=0, quant_max_bound=0, quant_min_bound=0):
    """``act(x + bias)`` in one pass (fused_bias_act.py; kernel paddle/phi/kernels/fusion/gpu/fused_bias_act_kernel.cu).
    The int8 dequantise / quantise arguments of the reference are not provided."""
    if dequant_scales is not None or shift is not None or smooth is not None or quant_scale > 0:
        raise NotImplementedError("fused_bias_act: the int8 (de)quantisation arguments are not provided")
    from ....ops import native
    needs_grad = torch.is_grad_enabled() and any(isinstance(t, torch.Tensor) and t.requires_grad for t in (x, bias))
    if (not needs_grad and _kernel_ok(x) and x.is_contiguous() and act_method in native.BIAS_ACT_CODES
            and (x.shape[-1] // (2 if act_method in ("swiglu", "geglu") else 1)) % 8 == 0
            and (bias is None or (_kernel_ok(bias) and bias.is_contiguous()))):
        return as_tensor(native.bias_act(x, bias, act_method))
    if bias is not None:
        x = x + bias
    return _act(act_method)(x)


def fused_dropout_add(x, y, p=0.5, training=True, mode="upscale_in_train", name=None):
    """``dropout(x) + y`` (fused_dropout_add.py:30).  On the GPU one Philox kernel does both and the backward pass
    regenerates the mask from (seed, offset) instead of reading a stored one."""
    if training and 0.0 < p < 1.0 and K.dropout_add_supported(x, y):
        return K.dropout_add(x, y, p, mode == "upscale_in_train")[0]
    return F.dropout(x, p, training=training, mode=mode) + y


def fused_bias_dropout_residual_layer_norm(x, residual, bias=None, ln_scale=None, ln_bias=None, dropout_rate=0.5,
                                           ln_epsilon=1e-5, training=True, mode="upscale_in_train", name=None):
    h = x if bias is None else x + bias
    h = residual + F.dropout(h, dropout_rate, training=training, mode=mode)
    return F.layer_norm(h, [h.shape[-1]], ln_scale, ln_bias, ln_epsilon)


def fused_feedforward(x, linear1_weight, linear2_weight, linear1_bias=None, linear2_bias=None, ln1_scale=None,
                      ln1_bias=None, ln2_scale=None, ln2_bias=None, dropout1_rate=0.5, dropout2_rate=0.5,
                      activation="relu", ln1_epsilon=1e-5, ln2_epsilon=1e-5, pre_layer_norm=False, training=True,
                      mode="upscale_in_train", ring_id=-1, add_residual=True, name=None):
    residual = x
    h = F.layer_norm(x, [x.shape[-1]], ln1_scale, ln1_bias, ln1_epsilon) if pre_layer_norm else x
    h = F.dropout(_act(activation)(F.linear(h, linear1_weight, linear1_bias)), dropout1_rate, training=training, mode=mode)
    h = F.linear(h, linear2_weight, linear2_bias)
    if ring_id >= 0:
        from ....distributed import collective as C
        C.all_reduce(h)
    h = F.dropout(h, dropout2_rate, training=training, mode=mode)
    if add_residual:
        h = residual + h
    if not pre_layer_norm:
        h = F.layer_norm(h, [h.shape[-1]], ln2_scale, ln2_bias, ln2_epsilon)
    return h


def fused_multi_head_attention(x, qkv_weight, linear_weight, pre_layer_norm=False, pre_ln_scale=None, pre_ln_bias=None,
                               ln_scale=None, ln_bias=None, pre_ln_epsilon=1e-5, qkv_bias=None, linear_bias=None,
                               cache_kv=None, attn_mask=None, dropout_rate=0.5, attn_dropout_rate=0.5,
                               ln_epsilon=1e-5, training=True, mode="upscale_in_train", ring_id=-1, add_residual=True,
                               num_heads=-1, transpose_qkv_wb=False, name=None):
    """qkv_weight ``[3, num_heads, head_dim, embed_dim]`` (or ``[embed_dim, 3*embed_dim]`` with
    ``transpose_qkv_wb``); self-attention with optional additive mask (fused_transformer.py:514)."""
    B, S, E = x.shape
    residual = x
    h = F.layer_norm(x, [E], pre_ln_scale, pre_ln_bias, pre_ln_epsilon) if pre_layer_norm else x
    if transpose_qkv_wb:
        nh = num_heads
        qkv = F.linear(h, qkv_weight, qkv_bias).reshape([B, S, 3, nh, E // nh])
    else:
        nh, hd = qkv_weight.shape[1], qkv_weight.shape[2]
        w = qkv_weight.reshape([3 * nh * hd, E]).t()
        b = qkv_bias.reshape([-1]) if qkv_bias is not None else None
        qkv = F.linear(h, w, b).reshape([B, S, 3, nh, hd])
    q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))     # [B, nh, S, hd]
    new_cache = None
    if cache_kv is not None:
        k = torch.cat([cache_kv[0], k], dim=2)
        v = torch.cat([cache_kv[1], v], dim=2)
        new_cache = as_tensor(torch.stack([k, v]))
    scores = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(q.shape[-1])
    if attn_mask is not None:
        scores = scores + attn_mask
    p = F.dropout(torch.softmax(scores, -1), attn_dropout_rate, training=training, mode=mode)
    o = torch.matmul(p, v).transpose(1, 2).reshape(B, S, -1)
    o = F.linear(as_tensor(o), linear_weight, linear_bias)
    if ring_id >= 0:
        from ....distributed import collective as C
        C.all_reduce(o)
    o = F.dropout(o, dropout_rate, training=training, mode=mode)
    if add_residual:
        o = residual + o
    if not pre_layer_norm:
        o = F.layer_norm(o, [E], ln_scale, ln_bias, ln_epsilon)
    return (o, new_cache) if cache_kv is not None else o


def variable_length_memory_efficient_attention(query, key, value, seq_lens, kv_seq_lens, mask=None, scale=None,
                                               causal=False, pre_cache_length=0):
    """query ``[B, H, Sq, D]``, key/value ``[B, Hkv, Sk, D]``; rows beyond ``seq_lens`` / keys beyond
    ``kv_seq_lens`` are ignored."""
    B, H, Sq, D = query.shape
    Hkv, Sk = key.shape[1], key.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if Hkv != H:
        key, value = (t.repeat_interleave(H // Hkv, 1) for t in (key, value))
    s = torch.matmul(query.float(), key.float().transpose(-1, -2)) * scale
    if mask is not None:
        s = s + mask.float()
    kpos = torch.arange(Sk, device=s.device)[None, None, None, :]
    valid = kpos < kv_seq_lens.reshape(B, 1, 1, 1)
    if causal:
        qpos = torch.arange(Sq, device=s.device)[None, None, :, None]
        valid = valid & (kpos <= qpos + (kv_seq_lens.reshape(B, 1, 1, 1) - seq_lens.reshape(B, 1, 1, 1)))
    s = s.masked_fill(~valid, float("-inf"))
    p = torch.nan_to_num(torch.softmax(s, -1), nan=0.0)
    return as_tensor(torch.matmul(p, value.float()).to(query.dtype))


def masked_multihead_attention(x, cache_kv=None, bias=None, src_mask=None, cum_offsets=None, sequence_lengths=None,
                               rotary_tensor=None, beam_cache_offset=None, qkv_out_scale=None, out_shift=None,
                               out_smooth=None, seq_len=1, rotary_emb_dims=0, use_neox_rotary_style=False,
                               compute_dtype="default", out_scale=-1, quant_round_type=1, quant_max_bound=127.0,
                               quant_min_bound=-127.0):
    """One decode step against a dense cache (masked_multihead_attention.py:74).  ``x`` ``[B, 3*H*D]``,
    ``cache_kv`` ``[2, B, H, max_seq, D]`` updated in place at position ``sequence_lengths[b]`` (or the length
    implied by ``src_mask``).  Returns ``(out [B, H*D], cache_kv)``."""
    two, B, H, max_seq, D = cache_kv.shape
    qkv = x if bias is None else x + bias.reshape([-1])
    qkv = qkv.reshape([B, 3, H, D])
    q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
    if sequence_lengths is not None:
        pos = sequence_lengths.reshape([-1]).to(torch.int64)
    else:
        pos = torch.full((B,), src_mask.shape[-1] - 1, dtype=torch.int64, device=x.device)
    if rotary_tensor is not None and rotary_emb_dims > 0:
        rt = rotary_tensor.reshape([2, B, -1, D]).float()
        cos, sin = rt[0, :, 0], rt[1, :, 0]

        def rot(t):
            tf = t.float()
            if use_neox_rotary_style:
                x1, x2 = tf[..., : D // 2], tf[..., D // 2:]
                r = torch.cat([-x2, x1], -1)
            else:
                r = torch.stack([-tf[..., 1::2], tf[..., 0::2]], -1).reshape(tf.shape)
            return (tf * cos[:, None] + r * sin[:, None]).to(t.dtype)
        q, k = rot(q), rot(k)
    idx = pos.reshape(B, 1, 1, 1).expand(B, H, 1, D)
    with torch.no_grad():
        raw = cache_kv.as_subclass(torch.Tensor)
        torch.Tensor.scatter_(raw[0], 2, idx, k.reshape(B, H, 1, D).as_subclass(torch.Tensor).to(raw.dtype))
        torch.Tensor.scatter_(raw[1], 2, idx, v.reshape(B, H, 1, D).as_subclass(torch.Tensor).to(raw.dtype))
    keys, vals = cache_kv[0].float(), cache_kv[1].float()
    s = torch.einsum("bhd,bhsd->bhs", q.float(), keys) / math.sqrt(D)
    valid = torch.arange(max_seq, device=x.device)[None, None, :] <= pos.reshape(B, 1, 1)
    if src_mask is not None:
        m = src_mask.reshape(B, 1, -1).float()
        s[..., : m.shape[-1]] = s[..., : m.shape[-1]] + m
    s = s.masked_fill(~valid, float("-inf"))
    o = torch.einsum("bhs,bhsd->bhd", torch.softmax(s, -1), vals).to(x.dtype)
    return as_tensor(o.reshape(B, H * D)), cache_kv


def blha_get_max_len(seq_lens_encoder, seq_lens_decoder, batch_size):
    return as_tensor(seq_lens_encoder.max().reshape([1])), as_tensor(seq_lens_decoder.max().reshape([1]))


def block_multihead_attention(qkv, key_cache, value_cache, seq_lens_encoder, seq_lens_decoder, seq_lens_this_time,
                              padding_offsets=None, cum_offsets=None, cu_seqlens_q=None, cu_seqlens_k=None,
                              block_tables=None, pre_key_cache=None, pre_value_cache=None, cache_k_quant_scales=None,
                              cache_v_quant_scales=None, cache_k_dequant_scales=None, cache_v_dequant_scales=None,
                              qkv_out_scale=None, qkv_bias=None, out_shift=None, out_smooth=None, max_enc_len_this_time=None,
                              max_dec_len_this_time=None, rope_emb=None, mask=None, tgt_mask=None, max_seq_len=-1,
                              block_size=64, use_neox_style=False, use_dynamic_cachekv_quant=False,
                              quant_round_type=1, quant_max_bound=127.0, quant_min_bound=-127.0, out_scale=-1,
                              compute_dtype="default", rope_theta=10000.0):
    """Paged attention over ``key_cache/value_cache [max_blocks, kv_heads, block_size, head_dim]``
    (block_multihead_attention.py:33).  ``qkv`` is ``[tokens, (Hq + 2 Hkv) * D]`` without padding; a batch is
    either all prefill (``seq_lens_encoder > 0``) or all decode (``seq_lens_decoder > 0``, one token each).
    Rotary embedding (half-rotation when ``use_neox_style``) is applied when ``rope_emb`` ``[2, 1, S, 1, D/2]`` is
    given.  Returns ``(out, qkv, key_cache, value_cache)``; the caches are updated in place."""
    from ....ops import attention as A
    from ....ops import native
    Hkv, D = key_cache.shape[1], key_cache.shape[3]
    Hq = qkv.shape[-1] // D - 2 * Hkv
    B = block_tables.shape[0]
    dec = bool((seq_lens_decoder.reshape([-1]) > 0).any()) and not bool((seq_lens_encoder.reshape([-1]) > 0).any())
    scale = 1.0 / math.sqrt(D)
    if qkv_bias is not None:
        qkv = qkv + qkv_bias
    use_native = qkv.is_cuda and qkv.dtype == torch.bfloat16 and D == 128 and block_size == 64 and \
        K.get_kernel_policy() == "fused"
    cos = sin = None
    if rope_emb is not None:
        re = rope_emb.reshape([2, -1, rope_emb.shape[-1]]).float()
        cos, sin = re[0].contiguous(), re[1].contiguous()          # [S, D/2]
    if dec:
        lens = seq_lens_decoder.reshape([-1]).to(torch.int32)
        if use_native and (cos is not None) and use_neox_style:
            q = torch.empty((B, Hq, D), dtype=qkv.dtype, device=qkv.device)
            native.decode_qkv_prep(qkv.contiguous(), None, cos, sin, lens, block_tables, q, key_cache, value_cache, Hq, Hkv)
            out = native.paged_decode_attn(q, key_cache, value_cache, block_tables, lens, scale, len_offset=1)
            return as_tensor(out.reshape(B, Hq * D)), qkv, key_cache, value_cache
        return _block_attn_reference(qkv, key_cache, value_cache, lens, block_tables, Hq, Hkv, D, cos, sin,
                                     use_neox_style, scale, block_size, decode=True)
    lens = seq_lens_encoder.reshape([-1]).to(torch.int32)
    if use_native:
        return _block_attn_prefill_native(qkv, key_cache, value_cache, lens, block_tables, Hq, Hkv, D, cos, sin,
                                          use_neox_style, scale, block_size)
    return _block_attn_reference(qkv, key_cache, value_cache, lens, block_tables, Hq, Hkv, D, cos, sin, use_neox_style,
                                 scale, block_size, decode=False)


def _block_attn_prefill_native(qkv, kc, vc, lens, tables, Hq, Hkv, D, cos, sin, neox, scale, bs):
    """Prefill of paged attention without a host loop: positions and page slots of all prompt tokens are computed on
    the device, the rotated keys / values are scattered into the pages in one indexed store each, and the packed
    prompts are attended in ONE launch of the flash kernels with a causal document mask (flash_attn_unpadded)."""
    from ....nn.functional.flash_attention import flash_attn_unpadded
    dev = qkv.device
    lens64 = lens.to(torch.int64)
    cu = torch.zeros(lens64.numel() + 1, dtype=torch.int64, device=dev)
    cu[1:] = lens64.cumsum(0)
    total = qkv.shape[0]
    tok = torch.arange(total, device=dev)
    seq = torch.searchsorted(cu, tok, right=True) - 1
    pos = tok - cu[seq]
    row = qkv.reshape(total, Hq + 2 * Hkv, D)
    q, k, v = row[:, :Hq], row[:, Hq:Hq + Hkv], row[:, Hq + Hkv:]
    if cos is not None:
        c, s_ = cos[pos][:, None, :], sin[pos][:, None, :]
        q = _rot(q.float(), c, s_, neox).to(qkv.dtype)
        k = _rot(k.float(), c, s_, neox).to(qkv.dtype)
    blk = tables.to(torch.int64)[seq, pos // bs]
    kc[blk, :, pos % bs] = k.to(kc.dtype)
    vc[blk, :, pos % bs] = v.to(vc.dtype)
    cu32 = cu.to(torch.int32)
    out, _ = flash_attn_unpadded(q.contiguous(), k.contiguous(), v.contiguous(), cu32, cu32, 0, 0, scale, causal=True)
    return as_tensor(out.reshape(total, Hq * D)), qkv, kc, vc


def _rot(t, cos, sin, neox):
    """t [..., D] fp32; cos/sin broadcastable [..., D/2]."""
    D = t.shape[-1]
    if neox:
        x1, x2 = t[..., : D // 2], t[..., D // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)
    x1, x2 = t[..., 0::2], t[..., 1::2]
    return torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).reshape(t.shape)


def _block_attn_reference(qkv, kc, vc, lens, tables, Hq, Hkv, D, cos, sin, neox, scale, bs, decode):
    """Plain-operator form of paged attention (prefill writes whole prompts, decode appends one token)."""
    B = tables.shape[0]
    outs = []
    tok = 0
    G = Hq // Hkv
    for b in range(B):
        n = 1 if decode else int(lens[b])
        start = int(lens[b]) if decode else 0
        row = qkv[tok:tok + n].float().reshape(n, Hq + 2 * Hkv, D)
        tok += n
        q, k, v = row[:, :Hq], row[:, Hq:Hq + Hkv], row[:, Hq + Hkv:]
        if cos is not None:
            c, s_ = cos[start:start + n, None, :], sin[start:start + n, None, :]
            q, k = _rot(q, c, s_, neox), _rot(k, c, s_, neox)
        for i in range(n):
            pos = start + i
            blk = int(tables[b, pos // bs])
            kc[blk, :, pos % bs] = k[i].to(kc.dtype)
            vc[blk, :, pos % bs] = v[i].to(vc.dtype)
        total = start + n
        nblk = (total + bs - 1) // bs
        ids = tables[b, :nblk].long()
        keys = kc[ids].float().permute(1, 0, 2, 3).reshape(Hkv, nblk * bs, D)[:, :total]
        vals = vc[ids].float().permute(1, 0, 2, 3).reshape(Hkv, nblk * bs, D)[:, :total]
        keys, vals = keys.repeat_interleave(G, 0), vals.repeat_interleave(G, 0)
        s = torch.einsum("nhd,hsd->hns", q, keys) * scale
        qpos = torch.arange(start, start + n, device=s.device)[None, :, None]
        kpos = torch.arange(total, device=s.device)[None, None, :]
        s = s.masked_fill(kpos > qpos, float("-inf"))
        o = torch.einsum("hns,hsd->nhd", torch.softmax(s, -1), vals)
        outs.append(o.reshape(n, Hq * D))
    return as_tensor(torch.cat(outs).to(qkv.dtype)), qkv, kc, vc


def fused_multi_transformer(x, ln_scales, ln_biases, qkv_weights, qkv_biases, linear_weights, linear_biases,
                            ffn_ln_scales, ffn_ln_biases, ffn1_weights, ffn1_biases, ffn2_weights, ffn2_biases,
                            pre_layer_norm=True, epsilon=1e-5, residual_alpha=1.0, cache_kvs=None, beam_offset=None,
                            pre_caches=None, seq_lens=None, rotary_embs=None, time_step=None, attn_mask=None,
                            dropout_rate=0.0, rotary_emb_dims=0, activation="gelu", training=False,
                            mode="upscale_in_train", trans_qkvw=True, ring_id=-1, norm_type="layernorm",
                            use_neox_rotary_style=False, gqa_group_size=-1, name=None):
    """Whole decoder stack in one call (fused_transformer.py:1053).  ``cache_kvs[i]`` is ``[2, B, H, max_seq, D]``;
    with ``time_step`` (a 1-element tensor: tokens already cached) one token per sequence is decoded, otherwise the
    prompt is processed and written to the caches.  Returns ``out`` (and the caches when given)."""
    B, S, E = x.shape
    L = len(qkv_weights)
    h = x
    norm = (lambda t, w, b: K.rms_norm(t, w, epsilon)) if norm_type == "rmsnorm" else \
        (lambda t, w, b: F.layer_norm(t, [E], w, b, epsilon))
    act = _act(activation)
    step = int(time_step.reshape([-1])[0]) if time_step is not None else None
    for i in range(L):
        residual = h
        a = norm(h, ln_scales[i], ln_biases[i] if ln_biases else None) if pre_layer_norm else h
        w = qkv_weights[i]
        if trans_qkvw:
            nh, hd = w.shape[1], w.shape[2]
            w2 = w.reshape([3 * nh * hd, E]).t()
        else:
            nh, hd = w.shape[2], w.shape[3]
            w2 = w.reshape([E, 3 * nh * hd])
        qb = qkv_biases[i].reshape([-1]) if qkv_biases and qkv_biases[i] is not None else None
        qkv = F.linear(a, w2, qb).reshape([B, S, 3, nh, hd])
        q, k, v = (qkv[:, :, j].transpose(1, 2) for j in range(3))       # [B, nh, S, hd]
        if rotary_embs is not None and rotary_emb_dims > 0:
            start = step if step is not None else 0
            re = rotary_embs.reshape([2, B, -1, hd]).float()
            cos, sin = re[0][:, None, start:start + S], re[1][:, None, start:start + S]
            half = hd // 2

            def rot(t):
                tf = t.float()
                if use_neox_rotary_style:
                    r = torch.cat([-tf[..., half:], tf[..., :half]], -1)
                else:
                    r = torch.stack([-tf[..., 1::2], tf[..., 0::2]], -1).reshape(tf.shape)
                return (tf * cos + r * sin).to(t.dtype)
            q, k = rot(q), rot(k)
        if cache_kvs is not None:
            cache = cache_kvs[i]
            start = step if step is not None else 0
            with torch.no_grad():
                cache[0][:, :, start:start + S] = k
                cache[1][:, :, start:start + S] = v
            k, v = cache[0][:, :, :start + S], cache[1][:, :, :start + S]
        s = torch.matmul(q.float(), k.float().transpose(-1, -2)) / math.sqrt(hd)
        if attn_mask is not None:
            s = s + attn_mask.float()[..., : s.shape[-2], : s.shape[-1]]
        elif step is None and S > 1:
            s = s + torch.full((S, S), float("-inf"), device=s.device).triu(1)
        o = torch.matmul(torch.softmax(s, -1), v.float()).to(x.dtype).transpose(1, 2).reshape(B, S, nh * hd)
        o = F.linear(as_tensor(o), linear_weights[i], linear_biases[i] if linear_biases else None)
        if ring_id >= 0:
            from ....distributed import collective as C
            C.all_reduce(o)
        h = residual_alpha * residual + o if pre_layer_norm else norm(residual + o, ln_scales[i], ln_biases[i] if ln_biases else None)
        residual = h
        f = norm(h, ffn_ln_scales[i], ffn_ln_biases[i] if ffn_ln_biases else None) if pre_layer_norm else h
        f = act(F.linear(f, ffn1_weights[i], ffn1_biases[i] if ffn1_biases else None))
        f = F.linear(f, ffn2_weights[i], ffn2_biases[i] if ffn2_biases else None)
        if ring_id >= 0:
            from ....distributed import collective as C
            C.all_reduce(f)
        h = residual_alpha * residual + f if pre_layer_norm else norm(residual + f, ffn_ln_scales[i], ffn_ln_biases[i] if ffn_ln_biases else None)
    return (h, cache_kvs) if cache_kvs is not None else h


# --------------------------------------------------------------------------------------------- MoE (fused_moe.py)
def moe_dispatch(x, gating_output, moe_topk, group_moe=False, topk_only_mode=False):
    """Top-k routing: returns (permute_input, token_nums_per_expert, permute_indices_per_token, expert_scales,
    top_k_indices)."""
    T, E = gating_output.shape
    probs = torch.softmax(gating_output.float(), -1)
    scales, topk = torch.topk(probs, moe_topk, dim=-1)
    flat = topk.reshape(-1)
    order = torch.argsort(flat, stable=True)
    token_of = order // moe_topk
    permuted = x[token_of]
    counts = torch.bincount(flat, minlength=E)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    return as_tensor(permuted), as_tensor(counts), as_tensor(inv.reshape(T, moe_topk)), as_tensor(scales), as_tensor(topk)


def moe_ffn(permute_input, token_nums_per_expert, ffn1_weight, ffn2_weight, ffn1_bias=None, ffn1_scale=None,
            ffn2_scale=None, quant_method="None"):
    """Grouped expert FFN over tokens sorted by expert: ffn1 ``[E, H, 2F]`` (SwiGLU), ffn2 ``[E, F, H]``."""
    outs, start = [], 0
    counts = token_nums_per_expert.tolist()
    for e, n in enumerate(counts):
        xe = permute_input[start:start + n]
        start += n
        if n == 0:
            continue
        h = torch.matmul(xe, ffn1_weight[e])
        if ffn1_bias is not None:
            h = h + ffn1_bias[e]
        h = swiglu(as_tensor(h))
        outs.append(torch.matmul(h, ffn2_weight[e]))
    return as_tensor(torch.cat(outs) if outs else permute_input.new_zeros((0, ffn2_weight.shape[-1])))


def moe_reduce(ffn_out, expert_scales_float, permute_indices_per_token, top_k_indices, ffn2_bias=None,
               norm_topk_prob=False, routed_scaling_factor=1.0):
    T, k = permute_indices_per_token.shape
    w = expert_scales_float.float()
    if norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    g = ffn_out[permute_indices_per_token.reshape(-1)].reshape(T, k, -1).float()
    if ffn2_bias is not None:
        g = g + ffn2_bias[top_k_indices].float()
    return as_tensor((g * w[..., None]).sum(1).to(ffn_out.dtype) * routed_scaling_factor)


def fused_moe(x, gate_weight, ffn1_weight, ffn2_weight, ffn1_bias=None, ffn1_scale=None, ffn2_bias=None,
              ffn2_scale=None, quant_method="None", moe_topk=2, norm_topk_prob=True, group_moe=False):
    shape = x.shape
    x2 = x.reshape([-1, shape[-1]])
    gate = torch.matmul(x2.float(), gate_weight.float())
    permuted, counts, inv, scales, topk = moe_dispatch(x2, gate, moe_topk)
    out = moe_ffn(permuted, counts, ffn1_weight, ffn2_weight, ffn1_bias)
    return moe_reduce(out, scales, inv, topk, ffn2_bias, norm_topk_prob).reshape(shape)


def quantize_expert_weights_fp8(ffn_weight):
    """bf16 expert weights ``[E, K, N]`` -> (e4m3 ``[E, N, K]``, fp32 scales ``[E, K/128, N/128]``), 128 x 128 blocks."""
    from ....ops import native
    return native.fp8_quant_weight(ffn_weight.detach().contiguous())


def moe_ffn_fp8(permute_input, token_nums_per_expert, ffn1_q, ffn1_scale, ffn2_q, ffn2_scale):
    """Expert SwiGLU FFN with block-scaled fp8 GEMMs: activations are quantised per 1 x 128 block on the fly, weights
    come pre-quantised from :func:`quantize_expert_weights_fp8`; both grouped GEMMs run all experts in one launch."""
    from ....ops import native
    counts = token_nums_per_expert.to(torch.int32)
    offsets = torch.zeros(counts.numel() + 1, dtype=torch.int32, device=counts.device)
    offsets[1:] = torch.cumsum(counts, 0)
    xq, xs = native.fp8_quant_1x128(permute_input.contiguous())
    h = native.grouped_gemm_fp8(xq, xs, ffn1_q, ffn1_scale, offsets)
    a = native.swiglu_fwd(h)
    aq, as_ = native.fp8_quant_1x128(a)
    return as_tensor(native.grouped_gemm_fp8(aq, as_, ffn2_q, ffn2_scale, offsets))


# ------------------------------------------------------------------ gate attention / cuDNN-style attention
def fused_gate_attention(query, key=None, query_weight=None, key_weight=None, value_weight=None, qkv_weight=None,
                         gate_linear_weight=None, gate_linear_bias=None, out_linear_weight=None, out_linear_bias=None,
                         nonbatched_bias=None, attn_mask=None, has_gating=True, merge_qkv=True, use_flash_attn=False):
    """AlphaFold-style gated self / cross attention over ``[batch, msa, res, dim]``
    (python/paddle/incubate/nn/functional/fused_gate_attention.py:26): per-head projections, additive ``attn_mask``
    and ``nonbatched_bias`` on the logits, a sigmoid gate on the attended values, output projection.
    ``merge_qkv=True`` takes ``qkv_weight [3, heads, head_dim, q_dim]``; otherwise separate ``[dim, heads, head_dim]``
    weights and an optional ``key`` tensor."""
    q_data = query
    if merge_qkv:
        assert key is None and qkv_weight is not None
        m_data = q_data
        qkv = torch.einsum("nbqa,thca->tnbqhc", q_data, qkv_weight)
        q, k, v = qkv[0], qkv[1], qkv[2]
    else:
        m_data = key if key is not None else q_data
        q = torch.einsum("nbqa,ahc->nbqhc", q_data, query_weight)
        k = torch.einsum("nbka,ahc->nbkhc", m_data, key_weight)
        v = torch.einsum("nbka,ahc->nbkhc", m_data, value_weight)
    q = q * (q.shape[-1] ** -0.5)
    logits = torch.einsum("nbqhc,nbkhc->nbhqk", q, k)
    if attn_mask is not None:
        logits = logits + attn_mask
    if nonbatched_bias is not None:
        logits = logits + nonbatched_bias.unsqueeze(1)
    weights = torch.softmax(logits, -1)
    avg = torch.einsum("nbhqk,nbkhc->nbqhc", weights, v)
    if has_gating:
        gate = torch.einsum("nbqc,chv->nbqhv", q_data, gate_linear_weight) + gate_linear_bias
        avg = avg * torch.sigmoid(gate)
    out = torch.einsum("nbqhc,hco->nbqo", avg, out_linear_weight)
    return as_tensor(out + out_linear_bias if out_linear_bias is not None else out)


def fused_dot_product_attention(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False,
                                scaling_factor=None, training=True, name=None):
    """``[batch, seq, heads, dim]`` attention (fused_dot_product_attention.py:129); ``attn_mask`` is boolean or 0/1
    (nonzero = may attend) of shape ``[batch, 1 | heads, seq_q, seq_k]``.  Unmasked and causal calls without dropout
    run on this library's flash-attention kernel."""
    from ....nn.functional.flash_attention import _attention_math
    from ....ops import functional as K
    drop = dropout_p if training else 0.0
    if attn_mask is None and drop == 0.0:
        return as_tensor(K.flash_attention(query, key, value, is_causal, scaling_factor))
    mask = None
    if attn_mask is not None:
        mask = attn_mask if attn_mask.dtype == torch.bool else attn_mask != 0
        if is_causal:
            mask = mask & torch.ones(query.shape[1], key.shape[1], dtype=torch.bool, device=mask.device).tril()
    return as_tensor(_attention_math(query, key, value, mask, drop, is_causal, scaling_factor))


def cudnn_flash_attention(q, k, v, bias=None, cu_seqlen_q=None, cu_seqlen_k=None, scaling_factor=1.0,
                          dropout_prob=0.0, training=True, mask_type=None, bias_type=None, name=None):
    """fused_dot_product_attention.py:21: ``mask_type`` in (None, "causal", "padding", "padding_causal"); padding
    masks come from ``cu_seqlen_q`` / ``cu_seqlen_k`` (per-sequence valid lengths as prefix sums); ``bias`` is added
    to the logits when ``bias_type`` is "pre_scale_bias" / "post_scale_bias"."""
    from ....nn.functional.flash_attention import _attention_math
    from ....ops import functional as K
    causal = mask_type in ("causal", "padding_causal")
    drop = dropout_prob if training else 0.0
    if mask_type in (None, "causal") and bias is None and drop == 0.0:
        return as_tensor(K.flash_attention(q, k, v, causal, scaling_factor))
    B, Sq, Sk = q.shape[0], q.shape[1], k.shape[1]
    add = torch.zeros(B, 1, Sq, Sk, dtype=q.dtype, device=q.device)
    if mask_type in ("padding", "padding_causal"):
        lq = (cu_seqlen_q[1:] - cu_seqlen_q[:-1]).reshape(B, 1, 1, 1)
        lk = (cu_seqlen_k[1:] - cu_seqlen_k[:-1]).reshape(B, 1, 1, 1)
        ok = (torch.arange(Sq, device=q.device).reshape(1, 1, Sq, 1) < lq) & \
             (torch.arange(Sk, device=q.device).reshape(1, 1, 1, Sk) < lk)
        add = add.masked_fill(~ok, float("-inf"))
    if causal:
        tri = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).tril()
        add = add.masked_fill(~tri, float("-inf"))
    if bias is not None and bias_type in ("pre_scale_bias", "post_scale_bias"):
        add = add + (bias * scaling_factor if bias_type == "pre_scale_bias" else bias)
    out = _attention_math(q, k, v, add, drop, False, scaling_factor)
    return as_tensor(torch.nan_to_num(out))          # fully padded query rows produce zeros


def fused_linear_param_grad_add(x, dout, dweight=None, dbias=None, multi_precision=True, has_bias=True):
    """``dweight (+)= x^T dout`` and ``dbias (+)= sum(dout)`` accumulated into existing (fp32 when ``multi_precision``)
    buffers, created when absent (paddle/phi/ops/yaml/fused_ops.yaml:382; kernel
    paddle/phi/kernels/fusion/gpu/fused_linear_param_grad_add_kernel.cu:36).  bf16 operands with an fp32 ``dweight``
    run on the tcgen05 GEMM with its reduce-add epilogue, so no temporary dW is written."""
    from ....ops import native
    x2, d2 = x.reshape(-1, x.shape[-1]), dout.reshape(-1, dout.shape[-1])
    acc_dtype = torch.float32 if multi_precision else x.dtype
    if dweight is None:
        dweight = torch.zeros(x2.shape[1], d2.shape[1], dtype=acc_dtype, device=x.device)
    if (x.is_cuda and x2.dtype == torch.bfloat16 and d2.dtype == torch.bfloat16 and dweight.dtype == torch.float32
            and x2.shape[1] % 8 == 0 and d2.shape[1] % 8 == 0 and dweight.is_contiguous()):
        native.gemm(x2.contiguous(), d2.contiguous(), trans_a=True, out=dweight, accumulate=True)
    else:
        dweight.add_((x2.float().t() @ d2.float()).to(dweight.dtype))
    if has_bias:
        if dbias is None:
            dbias = torch.zeros(d2.shape[1], dtype=acc_dtype, device=x.device)
        dbias.add_(d2.float().sum(0).to(dbias.dtype))
    return as_tensor(dweight), (as_tensor(dbias) if has_bias else None)


def skip_layernorm(x, y, scale, bias, epsilon, begin_norm_axis):
    """``layer_norm(x + y)`` (paddle/phi/ops/yaml/fused_ops.yaml:787)."""
    from ....ops import functional as K
    s = x + y
    return as_tensor(K.layer_norm(s, s.shape[begin_norm_axis:], scale, bias, epsilon))


def fused_embedding_eltwise_layernorm(ids, embs, bias, scale, epsilon=1e-5):
    """Sum of several embedding lookups followed by layer norm over the hidden axis (fused_ops.yaml:363)."""
    from ....ops import functional as K
    acc = None
    for i, w in zip(ids, embs):
        e = torch.nn.functional.embedding(i.squeeze(-1) if i.dim() == 3 else i, w)
        acc = e if acc is None else acc + e
    return as_tensor(K.layer_norm(acc, acc.shape[-1:], scale, bias, epsilon))
