"""Standalone all-reduce / all-gather / reduce-scatter over symmetric memory (one kernel each, device-side epoch,
CUDA-graph replayable).  Meant for latency-bound message sizes (up to a few MB); larger tensors stay on NCCL."""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib
from ..ops._lib import c_int, c_int64, check, ptr, stream
from . import symm

U64x8 = ctypes.c_ulonglong * 8
WAIT_MS = 2000


class SymmCollectives:
    def __init__(self, group, max_row_bytes):
        n = group.nranks
        self.group, self.n = group, n
        self.row_pad = (int(max_row_bytes) + 255) // 256 * 256
        chunk = _lib.kernels().pd_symm_chunk_bytes()
        nchunks = (self.row_pad + chunk - 1) // chunk
        recv_bytes = 2 * n * self.row_pad
        self.off_cnt = recv_bytes
        self.block = symm.SymmBlock(self.off_cnt + nchunks * 4 + 256, group)
        v = self.block.peer_ptrs(0)
        self.p_recv = U64x8(*(v + [0] * (8 - len(v))))
        v = self.block.peer_ptrs(self.off_cnt)
        self.p_cnt = U64x8(*(v + [0] * (8 - len(v))))
        self.state = torch.zeros(2, dtype=torch.int32, device=self.block.local.device)
        self.seen = torch.zeros(nchunks, dtype=torch.int32, device=self.block.local.device)

    def _run(self, kind, src, dst, row_bytes):
        assert row_bytes <= self.row_pad, "message larger than the buffer this object was created for"
        assert src.is_contiguous() and dst.is_contiguous()
        rc = _lib.kernels().pd_symm_collective(
            c_int(kind), ptr(src), ptr(dst), c_int64(row_bytes), c_int64(self.row_pad),
            c_int(1 if src.dtype == torch.bfloat16 else 0), c_int(self.group.rank), c_int(self.n), self.p_recv, self.p_cnt,
            ptr(self.state), ptr(self.seen), c_int(WAIT_MS), ptr(_lib.status_buffer(src.device)), stream())
        check(rc, "pd_symm_collective")
        from ..ops import native
        native._count()
        return dst

    def all_reduce(self, x, out=None):
        assert x.dtype in (torch.bfloat16, torch.float32)
        out = torch.empty_like(x) if out is None else out
        return self._run(0, x, out, x.numel() * x.element_size())

    def all_gather(self, x, out=None):
        out = torch.empty((self.n * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device) if out is None else out
        return self._run(1, x, out, x.numel() * x.element_size())

    def reduce_scatter(self, x, out=None):
        assert x.dtype in (torch.bfloat16, torch.float32) and x.shape[0] % self.n == 0
        out = torch.empty((x.shape[0] // self.n, *x.shape[1:]), dtype=x.dtype, device=x.device) if out is None else out
        return self._run(2, x, out, out.numel() * out.element_size())
