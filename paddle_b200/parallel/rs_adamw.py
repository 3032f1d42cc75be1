"""Gradient reduce-scatter + scaling + partitioned AdamW as one kernel over symmetric memory.

``FusedRSAdamW(group, shard_numel)`` owns the receive buffer (two slots of ``nranks`` rows), the per-chunk arrival
counters and the device-side epoch.  ``step(grad_bucket, master, m, v, param_shard, ...)`` consumes this rank's full
fp32 gradient bucket ``[nranks * shard_numel]`` and updates the owned slice of the optimizer state; the caller then
all-gathers the refreshed parameter slices (or lets the next forward gather them)."""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib
from ..ops._lib import c_float, c_int, c_int64, check, ptr, stream
from . import symm

U64x8 = ctypes.c_ulonglong * 8
WAIT_MS = 4000


class FusedRSAdamW:
    def __init__(self, group, shard_numel):
        n = group.nranks
        self.group, self.n, self.shard = group, n, int(shard_numel)
        self.padded = (self.shard + 3) // 4 * 4
        chunk = _lib.kernels().pd_rs_adamw_chunk()
        self.chunks = (self.shard + chunk - 1) // chunk
        recv_bytes = 2 * n * self.padded * 4
        self.off_cnt = (recv_bytes + 255) // 256 * 256
        self.block = symm.SymmBlock(self.off_cnt + self.chunks * 4 + 256, group)
        vals = self.block.peer_ptrs(0)
        self.p_recv = U64x8(*(vals + [0] * (8 - len(vals))))
        vals = self.block.peer_ptrs(self.off_cnt)
        self.p_cnt = U64x8(*(vals + [0] * (8 - len(vals))))
        self.state = torch.zeros(2, dtype=torch.int32, device=self.block.local.device)

    def step(self, grad_bucket, master, m, v, param_shard, lr, beta1, beta2, eps, coeff, beta1_pow, beta2_pow,
             grad_scale=None, skip=None):
        assert grad_bucket.dtype == torch.float32 and grad_bucket.numel() == self.n * self.shard
        rc = _lib.kernels().pd_rs_adamw(
            ptr(grad_bucket), c_int64(self.shard), c_int64(self.padded), c_int(self.group.rank), c_int(self.n), self.p_recv,
            self.p_cnt, ptr(master), ptr(m), ptr(v), ptr(param_shard), c_float(lr), c_float(beta1), c_float(beta2),
            c_float(eps), c_float(coeff), c_float(beta1_pow), c_float(beta2_pow), ptr(grad_scale), ptr(skip),
            ptr(self.state), c_int(WAIT_MS), ptr(_lib.status_buffer(grad_bucket.device)), stream(), None)
        check(rc, "pd_rs_adamw")
        from ..ops import native
        native._count()

    def reduce(self, grad_bucket, grad_out, grad_scale=None):
        """Phase A of the two-phase form: push + reduce only.  ``grad_out`` (fp32 ``[shard]``) receives this rank's
        slice of the summed gradient times ``grad_scale``; the optimizer state is untouched, so the caller can take
        the global norm of the reduced gradient before it applies the update."""
        assert grad_bucket.dtype == torch.float32 and grad_bucket.numel() == self.n * self.shard
        assert grad_out.dtype == torch.float32 and grad_out.numel() == self.shard
        rc = _lib.kernels().pd_rs_adamw(
            ptr(grad_bucket), c_int64(self.shard), c_int64(self.padded), c_int(self.group.rank), c_int(self.n), self.p_recv,
            self.p_cnt, None, None, None, None, c_float(0.0), c_float(0.0), c_float(0.0), c_float(0.0), c_float(0.0),
            c_float(0.0), c_float(0.0), ptr(grad_scale), None, ptr(self.state), c_int(WAIT_MS),
            ptr(_lib.status_buffer(grad_bucket.device)), stream(), ptr(grad_out))
        check(rc, "pd_rs_adamw")
        from ..ops import native
        native._count()
