"""GEMM -> all-reduce as one kernel over symmetric memory (tensor-parallel decode projections).

``GemmAllReduce(group, N, m_cap)`` owns the receive buffer ``[2][nranks][m_cap][N]`` bf16, the per-slab counters
and the device-side epoch; ``__call__(x, w, residual)`` launches the kernel.  All state that changes between calls
lives in device memory, so calls can be captured in a CUDA graph."""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib
from ..ops._lib import c_int, check, ptr, stream
from . import symm

U64x8 = ctypes.c_ulonglong * 8
WAIT_MS = 2000
_sm = None


def _sms():
    global _sm
    if _sm is None:
        _sm = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm


def supported(group, N, M):
    return symm.supported() and group is not None and 1 < group.nranks <= 8 and N % 128 == 0 and M <= 128


class GemmAllReduce:
    def __init__(self, group, N, m_cap=128):
        n = group.nranks
        self.group, self.N, self.m_cap, self.n = group, N, m_cap, n
        self.max_splits = 4
        recv_bytes = 2 * n * self.max_splits * m_cap * N * 2
        self.off_cnt = (recv_bytes + 255) // 256 * 256
        self.block = symm.SymmBlock(self.off_cnt + (N // 128) * 4 + 256, group)
        vals = self.block.peer_ptrs(0)
        self.p_recv = U64x8(*(vals + [0] * (8 - len(vals))))
        vals = self.block.peer_ptrs(self.off_cnt)
        self.p_cnt = U64x8(*(vals + [0] * (8 - len(vals))))
        self.state = torch.zeros(2, dtype=torch.int32, device=self.block.local.device)
        # in-switch reduction (multimem.ld_reduce over the receive buffers) from 4 ranks up; PD_GEMM_AR_NVLS=0 / 1 forces
        import os
        want = os.environ.get("PD_GEMM_AR_NVLS")
        self.mc_recv = self.block.mc_ptr if (self.block.mc_ptr and (want == "1" or (want is None and n >= 4))) else 0

    def __call__(self, x, w, residual=None, out=None):
        M, K = x.shape
        # K slices so that about one wave of CTAs streams the weights (same value on every rank: K is the local K)
        tiles = self.N // 128
        splits = max(1, min(self.max_splits, _sms() // tiles, (K // 64) // 4))
        if out is None:
            out = torch.empty((M, self.N), dtype=torch.bfloat16, device=x.device)
        rc = _lib.kernels().pd_gemm_ar(ptr(x), ptr(w), ptr(out), ptr(residual), c_int(M), c_int(self.N), c_int(K),
                                       c_int(x.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)),
                                       c_int(self.group.rank), c_int(self.n), self.p_recv, self.p_cnt, c_int(self.m_cap),
                                       c_int(splits), ptr(self.state), c_int(WAIT_MS), ptr(_lib.status_buffer(x.device)), stream(),
                                       ctypes.c_ulonglong(self.mc_recv))
        check(rc, "pd_gemm_ar")
        from ..ops import native
        native._count()
        return out
