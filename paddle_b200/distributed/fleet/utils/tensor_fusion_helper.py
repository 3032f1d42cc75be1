"""Flat buffers for parameters / gradients (python/paddle/distributed/fleet/utils/tensor_fusion_helper.py:
``flatten_dense_tensors`` :94, ``fused_parameters`` :768, ``FusedCommBuffer`` :330, ``assign_group_by_size`` :49).
Views into one contiguous allocation let a whole group be reduced with one collective and updated by one
flat-buffer kernel."""
from __future__ import annotations

import ctypes

import torch

from ...._core.tensor import as_tensor
from ... import collective as C

ALIGN = {torch.float32: 64, torch.float16: 128, torch.bfloat16: 128}     # elements per 256-byte boundary


class HOOK_ACTION:
    ALL_REDUCE, REDUCE, REDUCE_SCATTER = 0, 1, 2


def assign_group_by_size(parameters, group_size=128 * 1024 * 1024):
    """Bucket parameters (in order) so that each bucket holds at most ``group_size`` bytes; dtypes are not mixed.
    The split is computed by the native runtime."""
    from ....ops import _lib
    n = len(parameters)
    if n == 0:
        return {}
    sizes = (ctypes.c_int64 * n)(*[p.numel() * p.element_size() for p in parameters])
    kinds = (ctypes.c_int * n)(*[{torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}.get(p.dtype, 3) for p in parameters])
    out = (ctypes.c_int * n)()
    limits = (ctypes.c_int64 * 1)(int(group_size))
    _lib.runtime().pd_assign_group_by_size(sizes, kinds, ctypes.c_int(n), limits, ctypes.c_int(1), out)
    groups = {}
    for p, g in zip(parameters, out):
        groups.setdefault(int(g), []).append(p)
    return groups


def flatten_dense_tensors(parameters, use_main_grad=False, fuse_param=True, warp_buffer=False):
    """Returns (param_storage or None, grad_storage): parameters (and their gradients) re-pointed into flat
    buffers, each tensor starting on a 256-byte boundary."""
    dtype = parameters[0].dtype
    gdtype = torch.float32 if use_main_grad else dtype
    align = ALIGN.get(dtype, 64)
    offs, total = [], 0
    for p in parameters:
        offs.append(total)
        total += (p.numel() + align - 1) // align * align
    dev = parameters[0].device
    pbuf = torch.zeros(total, dtype=dtype, device=dev) if fuse_param else None
    gbuf = torch.zeros(total, dtype=gdtype, device=dev)
    with torch.no_grad():
        for p, o in zip(parameters, offs):
            n = p.numel()
            if fuse_param:
                pbuf[o:o + n].copy_(p.detach().reshape(-1))
                p.data = pbuf[o:o + n].view(p.shape)
            g = gbuf[o:o + n].view(p.shape)
            if use_main_grad:
                p.main_grad = as_tensor(g)
                p._main_grad_persistent = True
            else:
                p.grad = g
    return (as_tensor(pbuf) if fuse_param else None), as_tensor(gbuf)


class FusedCommBuffer:
    """One bucket: counts gradient arrivals, launches its collective when the last one is in
    (``add_grad`` / ``comm_grads`` / ``scale_grads``)."""

    def __init__(self, id, params, comm_group, acc_steps=1, act=HOOK_ACTION.ALL_REDUCE, dst=-1, use_main_grad=None,
                 fuse_param=False, scale_after_comm=True, release_grads=False):
        self._id, self._params, self._group, self._acc_steps, self._act, self._dst = id, params, comm_group, acc_steps, act, dst
        self.use_main_grad = use_main_grad if use_main_grad is not None else getattr(params[0], "main_grad", None) is not None
        self._scale_after_comm = scale_after_comm
        self.param_storage, self.grad_storage = flatten_dense_tensors(params, self.use_main_grad, fuse_param)
        self._checked_in, self._task = {}, None
        self._need = len(params) * acc_steps

    def add_grad(self, param, use_comm=True):
        self._checked_in[param.name] = self._checked_in.get(param.name, 0) + 1
        if sum(self._checked_in.values()) == self._need and use_comm:
            self.comm_grads()

    def comm_grads(self):
        g = self.grad_storage
        n = self._group.nranks if self._group is not None else 1
        if not self._scale_after_comm and n > 1:
            g.div_(n)
        if n > 1:
            if self._act == HOOK_ACTION.ALL_REDUCE:
                self._task = C.all_reduce(g, group=self._group, sync_op=False)
            elif self._act == HOOK_ACTION.REDUCE:
                self._task = C.reduce(g, dst=self._dst, group=self._group, sync_op=False)
            else:
                shard = g.numel() // n
                r = self._group.rank
                self._task = C.reduce_scatter(g[r * shard:(r + 1) * shard], list(g.chunk(n)), group=self._group, sync_op=False)

    def scale_grads(self):
        if self._task is not None:
            self._task.wait()
            self._task = None
        n = self._group.nranks if self._group is not None else 1
        if self._scale_after_comm and n > 1:
            self.grad_storage.div_(n)
        self._checked_in = {}


def fused_parameters(parameters, use_main_grad=False, fuse_param=True, comm_overlap=False, comm_group=None, act=None,
                     dst=-1, acc_step=1, scale_after_comm=False, group_params=False, apply_decay_param_fun=None,
                     group_size=128 * 1024 * 1024):
    """Bucket ``parameters`` and flatten each bucket.  Returns (decay_fused, all_fused, comm_buffers)."""
    buffers, fused = [], []
    for gid, ps in sorted(assign_group_by_size(list(parameters), group_size).items()):
        if comm_overlap:
            buf = FusedCommBuffer(gid, ps, comm_group, acc_step, act if act is not None else HOOK_ACTION.ALL_REDUCE, dst,
                                  use_main_grad, fuse_param, scale_after_comm)
            buffers.append(buf)
            fused.append(buf.param_storage if fuse_param else buf.grad_storage)
        else:
            pbuf, gbuf = flatten_dense_tensors(ps, use_main_grad, fuse_param)
            fused.append(pbuf if fuse_param else gbuf)
    decay = [f for f in fused] if apply_decay_param_fun is None else []
    return decay, fused, buffers
