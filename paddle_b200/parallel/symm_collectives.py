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
        self._nvls = None

    # ---- in-switch (NVLS) all-reduce for bandwidth-bound sizes
    NVLS_MAX_BLOCKS = 512
    NVLS_MIN_BYTES = int(__import__("os").environ.get("PD_SYMM_NVLS_MIN_BYTES", 512 << 10))

    def _nvls_state(self):
        if self._nvls is None:
            k = _lib.kernels()
            k.pd_symm_nvls_block_bytes.restype = c_int64
            bb = int(k.pd_symm_nvls_block_bytes(c_int64(self.row_pad), c_int(self.n)))
            nbuf = (self.row_pad + bb - 1) // bb * bb
            blk = symm.SymmBlock(nbuf + 2 * self.NVLS_MAX_BLOCKS * 4 + 256, self.group)
            v = blk.peer_ptrs(nbuf)
            self._nvls = {"block": blk, "cnt": U64x8(*(v + [0] * (8 - len(v)))),
                          "seen": torch.zeros(2 * self.NVLS_MAX_BLOCKS, dtype=torch.int32, device=blk.local.device)}
        return self._nvls

    def nvls_available(self):
        return self.n > 1 and symm.multicast_enabled() and self.block.mc_ptr != 0

    def _nvls_pays(self, nbytes):
        """Through the switch every GPU moves about (1 + 1/n) of the vector per direction (its own copy is read over
        the link as well), a direct exchange 2 (n - 1) / n: the switch only wins from four ranks up."""
        return self.n >= 4 and nbytes >= self.NVLS_MIN_BYTES and nbytes % 16 == 0 and self.nvls_available()

    def all_reduce_nvls(self, x, out=None):
        """Two-shot all-reduce in which the NVSwitch does the additions (multimem.ld_reduce) and the broadcast
        (multimem.st).  bf16 or fp32, byte size a multiple of 16."""
        assert x.dtype in (torch.bfloat16, torch.float32) and x.is_contiguous()
        out = torch.empty_like(x) if out is None else out
        nbytes = x.numel() * x.element_size()
        assert nbytes <= self.row_pad, "message larger than the buffer this object was created for"
        st = self._nvls_state()
        blk = st["block"]
        if blk.mc_ptr == 0:
            raise RuntimeError("this fabric offers no multicast mapping (NVLS) for symmetric memory")
        rc = _lib.kernels().pd_symm_all_reduce_nvls(
            ptr(x), ptr(out), c_int64(nbytes), c_int(1 if x.dtype == torch.bfloat16 else 0), ptr(blk.local),
            ctypes.c_ulonglong(blk.mc_ptr), c_int(self.group.rank), c_int(self.n), st["cnt"], c_int(self.NVLS_MAX_BLOCKS),
            ptr(st["seen"]), c_int(WAIT_MS), ptr(_lib.status_buffer(x.device)), stream())
        check(rc, "pd_symm_all_reduce_nvls")
        from ..ops import native
        native._count()
        return out

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
        nbytes = x.numel() * x.element_size()
        if self._nvls_pays(nbytes):
            return self.all_reduce_nvls(x, out)
        return self._run(0, x, out, nbytes)

    def all_gather(self, x, out=None):
        out = torch.empty((self.n * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device) if out is None else out
        return self._run(1, x, out, x.numel() * x.element_size())

    def reduce_scatter(self, x, out=None):
        assert x.dtype in (torch.bfloat16, torch.float32) and x.shape[0] % self.n == 0
        out = torch.empty((x.shape[0] // self.n, *x.shape[1:]), dtype=x.dtype, device=x.device) if out is None else out
        return self._run(2, x, out, out.numel() * out.element_size())

    def all_to_all(self, x, out=None):
        """Equal-split all-to-all: ``x [n * m, ...]``, rows ``[d * m, (d + 1) * m)`` go to rank d; the result holds the
        slices received from ranks 0 .. n-1 in that order (``alltoall_single`` without split sizes)."""
        assert x.shape[0] % self.n == 0
        out = torch.empty_like(x) if out is None else out
        return self._run(3, x, out, x.numel() * x.element_size() // self.n)
