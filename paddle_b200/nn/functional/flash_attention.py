"""Attention API (python/paddle/nn/functional/flash_attention.py: ``flash_attention:358``,
``scaled_dot_product_attention:1139``, ``flashmask_attention:1299``).  Layout is
``[batch, seq, heads, head_dim]`` as in the reference."""
from __future__ import annotations

import contextlib
import math

import torch

from ...ops import functional as K


@contextlib.contextmanager
def sdp_kernel(enable_math=False, enable_flash=True, enable_mem_efficient=True):
    yield


def flash_attention(query, key, value, dropout=0.0, causal=False, return_softmax=False, *, fixed_seed_offset=None,
                    rng_name="", training=True, name=None):
    if dropout > 0.0 and training:
        out = _attention_math(query, key, value, None, dropout, causal)
    else:
        out = K.flash_attention(query, key, value, causal)
    return out, None


def _attention_math(q, k, v, mask, dropout, causal, scale=None):
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if kh.shape[1] != qh.shape[1]:
        rep = qh.shape[1] // kh.shape[1]
        kh, vh = kh.repeat_interleave(rep, 1), vh.repeat_interleave(rep, 1)
    o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, dropout_p=dropout,
                                                         is_causal=causal and mask is None, scale=scale)
    return o.transpose(1, 2)


def scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, training=True,
                                 name=None):
    if attn_mask is None and (dropout_p == 0.0 or not training):
        return K.flash_attention(query, key, value, is_causal)
    return _attention_math(query, key, value, attn_mask, dropout_p if training else 0.0, is_causal)


def flash_attn_unpadded(query, key, value, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale,
                        dropout=0.0, causal=False, return_softmax=False, fixed_seed_offset=None, rng_name="",
                        training=True, name=None):
    """Variable-length attention over packed ``[total_tokens, heads, dim]`` tensors: each sequence is
    attended independently."""
    outs = []
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    for i in range(len(cq) - 1):
        q = query[cq[i]:cq[i + 1]].unsqueeze(0)
        k = key[ck[i]:ck[i + 1]].unsqueeze(0)
        v = value[ck[i]:ck[i + 1]].unsqueeze(0)
        outs.append(K.flash_attention(q, k, v, causal, scale).squeeze(0))
    return torch.cat(outs, 0), None


def flashmask_attention(query, key, value, startend_row_indices=None, *, dropout=0.0, causal=False,
                        window_size=None, return_softmax_lse=False, return_seed_offset=False,
                        fixed_seed_offset=None, rng_name="", training=True, name=None):
    """Column-sparse masked attention.  ``startend_row_indices`` is ``[b, h|1, s_k, {1,2,4}]``: for key
    column j, query rows in [start_j, end_j) of the lower (and optionally upper) triangle are masked."""
    if startend_row_indices is None:
        return K.flash_attention(query, key, value, causal)
    b, sq = query.shape[0], query.shape[1]
    sk = key.shape[1]
    idx = startend_row_indices
    rows = torch.arange(sq, device=query.device).view(1, 1, sq, 1)
    n = idx.shape[-1]
    lt_start = idx[..., 0].unsqueeze(2)  # [b, h, 1, sk]
    if causal:
        masked = rows >= lt_start
        if n == 2:
            masked = masked & (rows < idx[..., 1].unsqueeze(2))
        masked = masked | (rows < torch.arange(sk, device=query.device).view(1, 1, 1, sk) - (sk - sq))
    else:
        if n == 2:
            masked = (rows >= lt_start) | (rows < idx[..., 1].unsqueeze(2))
        else:
            masked = ((rows >= lt_start) & (rows < idx[..., 1].unsqueeze(2))) | (
                (rows >= idx[..., 2].unsqueeze(2)) & (rows < idx[..., 3].unsqueeze(2)))
    mask = torch.zeros(masked.shape, dtype=query.dtype, device=query.device).masked_fill(masked, float("-inf"))
    return _attention_math(query, key, value, mask, dropout if training else 0.0, False)


def calc_reduced_attention_scores(query, key, softmax_lse):
    """``sum over queries of softmax(Q K^T / sqrt(d))`` -> ``[batch, heads, 1, seq_k]`` fp32
    (python/paddle/nn/functional/flash_attention.py:2033), from the row log-sum-exp the attention forward returned
    (``[batch, heads, >= seq_q]``), so the probabilities are rebuilt one key block at a time and never stored whole."""
    b, sq, h, d = query.shape
    sk = key.shape[1]
    qh = query.transpose(1, 2).float() * (d ** -0.5)
    kh = key.transpose(1, 2).float()
    if kh.shape[1] != h:
        kh = kh.repeat_interleave(h // kh.shape[1], 1)
    lse = softmax_lse[:, :, :sq].float().unsqueeze(-1)
    out = torch.empty(b, h, 1, sk, dtype=torch.float32, device=query.device)
    blk = 2048
    for s0 in range(0, sk, blk):
        p = torch.exp(qh @ kh[:, :, s0:s0 + blk].transpose(-1, -2) - lse)
        out[:, :, 0, s0:s0 + blk] = p.sum(2)
    return out
