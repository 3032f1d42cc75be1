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


def _native_mask_ok(q, k, v):
    from ...ops import attention as A
    from ...ops.functional import _native
    return _native(q) and A.supported(q, k, v)


def flash_attn_unpadded(query, key, value, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale,
                        dropout=0.0, causal=False, return_softmax=False, fixed_seed_offset=None, rng_name="",
                        training=True, name=None):
    """Variable-length attention over packed ``[total_tokens, heads, dim]`` tensors: each sequence is
    attended independently (python/paddle/nn/functional/flash_attention.py:756).

    Self-attention over one packing (``cu_seqlens_q`` and ``cu_seqlens_k`` are the same tensor or equal) runs as ONE
    launch of the flash kernels on the packed tensor with a document mask built on the device from ``cu_seqlens`` -
    key column j is hidden from the rows outside its own sequence, and key tiles that lie outside a query tile's
    sequences are skipped - so nothing is read back to the host.  Otherwise one launch per sequence on views."""
    use_dropout = dropout > 0.0 and training
    same = cu_seqlens_q is cu_seqlens_k or (cu_seqlens_q.shape == cu_seqlens_k.shape and query.shape[0] == key.shape[0]
                                            and bool(torch.equal(cu_seqlens_q, cu_seqlens_k)))
    if same and not use_dropout and _native_mask_ok(query.unsqueeze(0), key.unsqueeze(0), value.unsqueeze(0)):
        from ...ops import attention as A
        total = query.shape[0]
        cu = torch.as_tensor(cu_seqlens_q, device=query.device).to(torch.int64)
        pos = torch.arange(total, device=query.device)
        seq = torch.searchsorted(cu, pos, right=True) - 1                # sequence of every token
        start, end = cu[seq], cu[seq + 1]
        if causal:
            idx = end.view(1, 1, total, 1)                               # rows from the end of j's sequence on: hidden
        else:
            idx = torch.stack([end, start], -1).view(1, 1, total, 2)     # [lts, ute]
        mask = A.normalize_flashmask(idx, causal, total)
        out = A.flash_attn_func(query.unsqueeze(0), key.unsqueeze(0), value.unsqueeze(0), causal, float(scale), mask)
        from ..._core.tensor import as_tensor
        return as_tensor(out.squeeze(0)), None
    outs = []
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    for i in range(len(cq) - 1):
        q = query[cq[i]:cq[i + 1]].unsqueeze(0)
        k = key[ck[i]:ck[i + 1]].unsqueeze(0)
        v = value[ck[i]:ck[i + 1]].unsqueeze(0)
        if use_dropout:
            outs.append(_attention_math(q, k, v, None, dropout, causal, scale).squeeze(0))
        else:
            outs.append(K.flash_attention(q, k, v, causal, scale).squeeze(0))
    return torch.cat(outs, 0), None


def flash_attn_varlen_func(query, key, value, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale=None,
                           dropout=0.0, causal=False, **kwargs):
    scale = scale if scale is not None else 1.0 / math.sqrt(query.shape[-1])
    return flash_attn_unpadded(query, key, value, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale,
                               dropout, causal, **kwargs)


def _flashmask_dense(idx, sq, sk, causal, device):
    rows = torch.arange(sq, device=device).view(1, 1, sq, 1)
    n = idx.shape[-1]
    lt_start = idx[..., 0].unsqueeze(2)  # [b, h, 1, sk]
    if causal:
        masked = rows >= lt_start
        if n == 2:
            masked = masked & (rows < idx[..., 1].unsqueeze(2))
        masked = masked | (rows < torch.arange(sk, device=device).view(1, 1, 1, sk) - (sk - sq))
    else:
        if n == 2:
            masked = (rows >= lt_start) | (rows < idx[..., 1].unsqueeze(2))
        else:
            masked = ((rows >= lt_start) & (rows < idx[..., 1].unsqueeze(2))) | (
                (rows >= idx[..., 2].unsqueeze(2)) & (rows < idx[..., 3].unsqueeze(2)))
    return masked


def flashmask_attention(query, key, value, startend_row_indices=None, *, dropout=0.0, causal=False,
                        window_size=None, return_softmax_lse=False, return_seed_offset=False,
                        fixed_seed_offset=None, rng_name="", training=True, name=None):
    """Column-sparse masked attention (python/paddle/nn/functional/flash_attention.py:1299).
    ``startend_row_indices`` is ``[b, h|1, s_k, {1,2,4}]``: for key column j, query rows in [start_j, end_j) of the
    lower (and optionally upper) triangle are masked.  ``window_size`` (int or (left, right)) adds a sliding window
    and is folded into the same bounds.  On the GPU the bounds are applied inside the flash kernels (forward and
    backward) and key tiles that are masked as a whole are not visited; with dropout, or for shapes the kernels do
    not take, the mask is materialised and the math path runs."""
    sq, sk = query.shape[1], key.shape[1]
    if window_size is not None:
        startend_row_indices = _window_bounds(startend_row_indices, window_size, causal, query.shape[0], sq, sk,
                                              query.device)
    if startend_row_indices is None:
        out = K.flash_attention(query, key, value, causal)
        return (out, None) if return_softmax_lse else out
    idx = startend_row_indices
    if not (dropout > 0.0 and training) and _native_mask_ok(query, key, value) and idx.shape[1] in (
            1, query.shape[2], key.shape[2]):
        from ..._core.tensor import as_tensor
        from ...ops import attention as A
        mask = A.normalize_flashmask(idx, causal, sq)
        out, lse = A.flash_attn_func(query, key, value, causal, 1.0 / math.sqrt(query.shape[-1]), mask, return_lse=True)
        out = as_tensor(out)
        return (out, as_tensor(lse)) if return_softmax_lse else out
    masked = _flashmask_dense(idx, sq, sk, causal, query.device)
    mask = torch.zeros(masked.shape, dtype=query.dtype, device=query.device).masked_fill(masked, float("-inf"))
    out = _attention_math(query, key, value, mask, dropout if training else 0.0, False)
    return (out, None) if return_softmax_lse else out


def _window_bounds(idx, window_size, causal, b, sq, sk, device):
    """Sliding window as flashmask bounds, merged with ``idx`` when both are given (the reference accepts only one of
    the two per call for non-trivial ``idx``; merging takes the tighter bound)."""
    left, right = (window_size, window_size) if isinstance(window_size, int) else window_size
    cols = torch.arange(sk, device=device, dtype=torch.int32)
    lts = (cols + left + 1).clamp(max=sq)                     # rows further down than `left` below the diagonal: hidden
    if causal:
        w = lts.view(1, 1, sk, 1).expand(b, 1, sk, 1)
        if idx is None:
            return w.contiguous()
        assert idx.shape[-1] == 1, "window_size can be combined with a one-bound causal flashmask only"
        return torch.minimum(idx.to(torch.int32), w.expand(idx.shape)).contiguous()
    ute = (cols - right).clamp(min=0)
    w = torch.stack([lts, ute], -1).view(1, 1, sk, 2).expand(b, 1, sk, 2)
    if idx is None:
        return w.contiguous()
    assert idx.shape[-1] == 2, "window_size can be combined with a [lts, ute] flashmask only"
    w = w.expand(idx.shape)
    return torch.stack([torch.minimum(idx[..., 0].to(torch.int32), w[..., 0]),
                        torch.maximum(idx[..., 1].to(torch.int32), w[..., 1])], -1).contiguous()


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
