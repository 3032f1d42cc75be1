"""Attention-bias descriptions for ``memory_efficient_attention`` (python/paddle/incubate/nn/attn_bias.py):
objects that say *which* (query, key) pairs may attend, materialised as an additive mask only when a kernel needs one.
Sequences packed along the token axis are described by ``SeqLenInfo`` (start offsets) and the block-diagonal masks
built from them."""
from __future__ import annotations

import math

import torch

from ..._core import dtype as _dt
from ..._core.tensor import as_tensor


def _neg_inf_mask(shape, dtype, keep):
    out = torch.zeros(shape, dtype=_dt.to_torch(dtype) or torch.float32)
    return out.masked_fill(~keep, float("-inf"))


class AttentionBias:
    def materialize(self, shape, dtype="float32"):
        raise NotImplementedError


class LowerTriangularMask(AttentionBias):
    """Causal mask: query i sees keys 0..i."""

    def materialize(self, shape, dtype="float32"):
        q, k = shape[-2], shape[-1]
        keep = torch.ones(q, k, dtype=torch.bool).tril()
        return as_tensor(_neg_inf_mask(shape, dtype, keep.expand(shape)))

    def add_bias(self, bias):
        return LowerTriangularMaskWithTensorBias(bias)


class LowerTriangularMaskWithTensorBias(LowerTriangularMask):
    def __init__(self, bias):
        self._bias = bias

    def materialize(self, shape, dtype="float32"):
        return as_tensor(super().materialize(shape, dtype).to(self._bias.device) + self._bias)


class SeqLenInfo:
    """Start offsets of sequences packed one after another: ``seqstart_py = [0, l0, l0 + l1, ...]``."""

    def __init__(self, seqstart, max_seqlen, seqstart_py):
        self.seqstart, self.max_seqlen, self.seqstart_py = seqstart, max_seqlen, seqstart_py

    def intervals(self):
        yield from zip(self.seqstart_py, self.seqstart_py[1:])

    @classmethod
    def from_seqlens(cls, seqlens):
        starts, mx = [0], 0
        for n in seqlens:
            mx = max(mx, n)
            starts.append(starts[-1] + n)
        return cls(as_tensor(torch.tensor(starts, dtype=torch.int32)), mx, starts)

    def split(self, x, batch_sizes=None):
        assert x.shape[0] == 1 and self.seqstart_py[-1] == x.shape[1]
        if batch_sizes is None:
            batch_sizes = [1] * (len(self.seqstart_py) - 1)
        out, i = [], 0
        for b in batch_sizes:
            lo, hi = self.seqstart_py[i], self.seqstart_py[i + b]
            out.append(x[:, lo:hi].reshape([b, -1, *x.shape[2:]]))
            i += b
        return out


class PaddedSeqLenInfo(SeqLenInfo):
    """Sequences stored in slots of a fixed ``padding`` length; ``seqlen_py`` holds the used length of every slot."""

    def __init__(self, seqstart, max_seqlen, seqstart_py, seqlen, seqlen_py):
        super().__init__(seqstart, max_seqlen, seqstart_py)
        self.seqlen, self.seqlen_py = seqlen, seqlen_py

    def intervals(self):
        for start, n in zip(self.seqstart_py, self.seqlen_py):
            yield start, start + n

    @classmethod
    def from_seqlens(cls, seqlens):
        raise NotImplementedError("use from_seqlens_padded")

    @classmethod
    def from_seqlens_padded(cls, seqlens, padding):
        assert all(n <= padding for n in seqlens)
        starts = list(range(0, len(seqlens) * padding + 1, padding))
        return cls(as_tensor(torch.tensor(starts, dtype=torch.int32)), max(seqlens), starts,
                   as_tensor(torch.tensor(seqlens, dtype=torch.int32)), list(seqlens))

    def split(self, x, batch_sizes=None):
        raise NotImplementedError


class BlockDiagonalMask(AttentionBias):
    """Every packed sequence attends only to itself."""

    def __init__(self, q_seqinfo, k_seqinfo, _batch_sizes=None):
        self.q_seqinfo, self.k_seqinfo, self._batch_sizes = q_seqinfo, k_seqinfo, _batch_sizes

    def _block_keep(self, q, k):
        return torch.ones(q, k, dtype=torch.bool)

    def materialize(self, shape, dtype="float32"):
        assert shape[-1] == self.k_seqinfo.seqstart_py[-1] and shape[-2] == self.q_seqinfo.seqstart_py[-1]
        keep = torch.zeros(shape[-2], shape[-1], dtype=torch.bool)
        for (qs, qe), (ks, ke) in zip(self.q_seqinfo.intervals(), self.k_seqinfo.intervals()):
            keep[qs:qe, ks:ke] = self._block_keep(qe - qs, ke - ks)
        return as_tensor(_neg_inf_mask(shape, dtype, keep.expand(shape)))

    @classmethod
    def from_seqlens(cls, q_seqlen, kv_seqlen=None):
        assert kv_seqlen is None or len(q_seqlen) == len(kv_seqlen)
        q = SeqLenInfo.from_seqlens(q_seqlen)
        k = q if kv_seqlen is None or list(q_seqlen) == list(kv_seqlen) else SeqLenInfo.from_seqlens(kv_seqlen)
        return cls(q, k)

    @classmethod
    def from_tensor_list(cls, tensors):
        sizes = [t.shape[0] for t in tensors]
        lens = []
        for t in tensors:
            lens += [t.shape[1]] * t.shape[0]
        mask = cls.from_seqlens(lens)
        mask._batch_sizes = sizes
        packed = torch.cat([t.reshape([1, -1, *t.shape[2:]]) for t in tensors], 1)
        return mask, as_tensor(packed)

    @classmethod
    def from_tensor_lists_qkv(cls, tensors_q, tensors_k, tensors_v=None):
        assert len(tensors_q) == len(tensors_k) and (tensors_v is None or len(tensors_v) == len(tensors_q))
        sizes, ql, kl = [], [], []
        for q, k in zip(tensors_q, tensors_k):
            assert q.shape[0] == k.shape[0]
            sizes.append(q.shape[0])
            ql += [q.shape[1]] * q.shape[0]
            kl += [k.shape[1]] * q.shape[0]
        mask = cls.from_seqlens(ql, kl)
        mask._batch_sizes = sizes

        def pack(ts):
            return as_tensor(torch.cat([t.reshape([1, -1, *t.shape[2:]]) for t in ts], 1))
        return mask, pack(tensors_q), pack(tensors_k), (pack(tensors_v) if tensors_v is not None else None)

    def split_queries(self, tensor):
        return self.q_seqinfo.split(tensor, self._batch_sizes)

    def split_kv(self, tensor):
        return self.k_seqinfo.split(tensor, self._batch_sizes)

    def split(self, tensor):
        assert self.q_seqinfo is self.k_seqinfo
        return self.q_seqinfo.split(tensor, self._batch_sizes)

    def make_causal(self):
        return BlockDiagonalCausalMask(self.q_seqinfo, self.k_seqinfo, self._batch_sizes)


class BlockDiagonalCausalMask(BlockDiagonalMask):
    def _block_keep(self, q, k):
        return torch.ones(q, k, dtype=torch.bool).tril()


class BlockDiagonalCausalWithOffsetPaddedKeysMask(AttentionBias):
    """Decoding against padded key slots: the queries of a sequence are its LAST tokens, so query i of n sees keys
    ``0 .. len_k - n + i``."""

    def __init__(self, q_seqinfo, k_seqinfo, causal_diagonal=None):
        self.q_seqinfo, self.k_seqinfo, self.causal_diagonal = q_seqinfo, k_seqinfo, causal_diagonal

    def materialize(self, shape, dtype="float32"):
        assert shape[-1] == self.k_seqinfo.seqstart_py[-1] and shape[-2] == self.q_seqinfo.seqstart_py[-1]
        keep = torch.zeros(shape[-2], shape[-1], dtype=torch.bool)
        for (qs, qe), (ks, ke) in zip(self.q_seqinfo.intervals(), self.k_seqinfo.intervals()):
            q, k = qe - qs, ke - ks
            keep[qs:qe, ks:ke] = torch.ones(q, k, dtype=torch.bool).tril(diagonal=k - q)
        return as_tensor(_neg_inf_mask(shape, dtype, keep.expand(shape)))

    @classmethod
    def from_seqlens(cls, q_seqlen, kv_padding, kv_seqlen, causal_diagonal=None):
        assert len(q_seqlen) == len(kv_seqlen)
        return cls(SeqLenInfo.from_seqlens(q_seqlen), PaddedSeqLenInfo.from_seqlens_padded(kv_seqlen, kv_padding),
                   causal_diagonal)
