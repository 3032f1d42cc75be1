"""``paddle.incubate.nn.memory_efficient_attention`` (python/paddle/incubate/nn/memory_efficient_attention.py:70):
attention over ``[batch, seq, heads, dim]`` with an ``attn_bias`` that is ``None``, a tensor, or one of the mask
descriptions of ``attn_bias``.  Plain causal / unmasked calls run on the tcgen05 flash-attention kernel, block-diagonal
masks as one flash-attention call per packed sequence, anything else through a materialised additive mask."""
from __future__ import annotations

import torch

from ..._core.tensor import as_tensor
from ...nn.functional.flash_attention import _attention_math
from ...ops import functional as K
from .attn_bias import (AttentionBias, BlockDiagonalCausalMask, BlockDiagonalCausalWithOffsetPaddedKeysMask,
                        BlockDiagonalMask, LowerTriangularMask, LowerTriangularMaskWithTensorBias)

SUPPORTED_ATTN_BIAS_TYPES = {type(None), torch.Tensor, LowerTriangularMask, LowerTriangularMaskWithTensorBias,
                             BlockDiagonalMask, BlockDiagonalCausalMask, BlockDiagonalCausalWithOffsetPaddedKeysMask}


def memory_efficient_attention(query, key, value, attn_bias=None, p=0.0, scale=None, training=True):
    if not (attn_bias is None or isinstance(attn_bias, (torch.Tensor, AttentionBias))):
        raise TypeError(f"unsupported attn_bias type {type(attn_bias).__name__}")
    drop = p if training else 0.0
    if drop == 0.0:
        if attn_bias is None or type(attn_bias) is LowerTriangularMask:
            return as_tensor(K.flash_attention(query, key, value, attn_bias is not None, scale))
        if type(attn_bias) in (BlockDiagonalMask, BlockDiagonalCausalMask) and query.shape[0] == 1:
            causal = type(attn_bias) is BlockDiagonalCausalMask
            outs = []
            for (qs, qe), (ks, ke) in zip(attn_bias.q_seqinfo.intervals(), attn_bias.k_seqinfo.intervals()):
                outs.append(K.flash_attention(query[:, qs:qe], key[:, ks:ke], value[:, ks:ke], causal, scale))
            return as_tensor(torch.cat(outs, 1))
    mask = attn_bias
    if isinstance(attn_bias, AttentionBias):
        shape = (query.shape[0], query.shape[2], query.shape[1], key.shape[1])
        mask = attn_bias.materialize(shape, "float32").to(device=query.device, dtype=query.dtype)
    return as_tensor(_attention_math(query, key, value, mask, drop, False, scale))
