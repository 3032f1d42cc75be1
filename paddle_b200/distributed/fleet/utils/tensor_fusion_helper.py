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


# ------------------------------------------------------------------ helpers used by the sharding optimizers
def get_current_device_type():
    return "gpu" if torch.cuda.is_available() else "cpu"


def get_grad_address(param, use_main_grad):
    """Device address of the gradient that would be communicated (``None`` when there is none yet)."""
    g = getattr(param, "main_grad", None) if use_main_grad else getattr(param, "grad", None)
    return None if g is None else g.data_ptr()


def bw_hook_func(buffer, param):
    """Backward hook that checks ``param``'s gradient in with its communication bucket."""
    @torch.no_grad()
    def fused_comm(*_):
        buffer.add_grad(param)
    return fused_comm


def filter_params(params, is_fp32, is_distributed, need_clip):
    """Parameters that are (not) fp32, (not) tensor-parallel-distributed and (not) subject to clipping; all of one
    dtype, which is returned with them (tensor_fusion_helper.py:830)."""
    out = [p for p in params
           if bool(getattr(p, "is_distributed", False)) == bool(is_distributed)
           and bool(getattr(p, "need_clip", True)) == bool(need_clip)
           and (p.dtype == torch.float32) == bool(is_fp32)]
    dtypes = {p.dtype for p in out}
    assert len(dtypes) <= 1, f"mixed dtypes in one filter class: {dtypes}"
    return out, (dtypes.pop() if dtypes else None)


def obtain_storage(parameters, use_main_grad=False, clip=True, dist=False, fuse_param=True, comm_overlap=False,
                   act=None, comm_group=None, dst=-1, acc_steps=1, scale_after_comm=False, use_reduce_avg=False,
                   group_size=256 * 1024 * 1024):
    """Buckets ``parameters`` and gives every bucket a ``FusedCommBuffer``; returns (flat parameter storages tagged with
    ``need_clip`` / ``is_distributed``, the buffers when ``comm_overlap`` registers their backward hooks)
    (tensor_fusion_helper.py:783)."""
    if not parameters:
        return [], []
    storage, buffers = [], []
    for gid, ps in sorted(assign_group_by_size(list(parameters), group_size).items()):
        buf = FusedCommBuffer(gid, ps, comm_group, acc_steps, act if act is not None else HOOK_ACTION.ALL_REDUCE, dst,
                              use_main_grad, fuse_param, scale_after_comm)
        if fuse_param:
            buf.param_storage.need_clip, buf.param_storage.is_distributed = clip, dist
            storage.append(buf.param_storage)
        if comm_overlap:
            for p in ps:
                p.register_hook(bw_hook_func(buf, p)) if p.requires_grad else None
            buffers.append(buf)
    return storage, buffers


class ShardingGradView:
    """One parameter's place inside a bucket whose flat buffers are cut into ``sharding_degree`` equal shards
    (tensor_fusion_helper.py:181): the parameter occupies ``[index, index + padded_size)``; this rank owns
    ``[rank * shard, (rank + 1) * shard)``; their overlap is the slice this rank updates.  The parameter's data is
    re-pointed into ``param_buffer`` and its gradient (or ``main_grad``) into ``grad_buffer``, so the bucket can be
    reduce-scattered and the owned slice updated in place."""

    def __init__(self, param, param_buffer, grad_buffer, index, padded_size, sharding_degree, rank,
                 use_main_grad=False, release_grad=False):
        self._param, self._param_buffer, self._grad_buffer = param, param_buffer, grad_buffer
        self._index, self._padded_size = index, padded_size
        self._sharding_degree, self._rank = sharding_degree, rank
        self._use_main_grad, self._release_grad = use_main_grad, release_grad
        shard = param_buffer.numel() // sharding_degree
        self._rank_begin = max(rank, 0) * shard
        self._param_begin = max(index, self._rank_begin)
        self._param_end = min(index + padded_size, self._rank_begin + shard)
        self._slice_grad = None
        n = param.numel()
        with torch.no_grad():
            param_buffer[index:index + n].copy_(param.detach().reshape(-1))
            param.data = param_buffer[index:index + n].view(param.shape)
        if not release_grad:
            self._link_grad_to_buffer()

    def _link_grad_to_buffer(self):
        n = self._param.numel()
        if self._param_begin < self._param_end:
            self._slice_grad = self._grad_buffer[self._param_begin:self._param_end]
        g = self._grad_buffer[self._index:self._index + n].view(self._param.shape)
        if self._use_main_grad:
            self._param.main_grad = as_tensor(g)
        else:
            self._param.grad = g

    def fill_slice_param(self, slice_param):
        """Points ``slice_param`` (1-D) at this rank's slice of the parameter inside the flat buffer."""
        slice_param.data = self._param_buffer[self._param_begin:max(self._param_end, self._param_begin)]

    def assign_slice_grad(self, slice_param):
        if self._slice_grad is None:
            return
        self.fill_slice_param(slice_param)
        if self._use_main_grad:
            slice_param.main_grad = as_tensor(self._slice_grad)
        else:
            slice_param.grad = self._slice_grad

    def _get_padding(self):
        """The part of this rank's gradient slice that lies in the parameter's alignment padding (must stay zero)."""
        if self._slice_grad is None:
            return None
        lo = max(self._param_begin, self._index + self._param.numel())
        hi = min(self._param_end, self._index + self._padded_size)
        if lo >= hi:
            return None
        return self._slice_grad[self._slice_grad.numel() - (hi - lo):]

    def _clear_grad_buffer(self):
        self._slice_grad = None
        self._grad_buffer = None
        if self._use_main_grad:
            self._param.main_grad = None
        else:
            self._param.grad = None

    def _reset_grad_buffer(self, grad_buffer=None):
        if grad_buffer is not None:
            self._grad_buffer = grad_buffer
        self._link_grad_to_buffer()


def build_reduce_scatter_buffer(parameters, sharding_degree, rank, use_main_grad=False, release_grad=False,
                                init_slice_param=False, slice_params=None):
    """Flat parameter / gradient buffers for one reduce-scatter bucket: every parameter padded to a 256-byte
    boundary, the total padded to a multiple of ``sharding_degree``; returns ({name: ShardingGradView}, total elements,
    param_buffer, grad_buffer) (tensor_fusion_helper.py:330)."""
    dtype = parameters[0].dtype
    align = ALIGN.get(dtype, 64)
    index, total = {}, 0
    for p in parameters:
        assert p.dtype == dtype, "one bucket holds one dtype"
        padded = (p.numel() + align - 1) // align * align
        index[p.name] = (total, padded)
        total += padded
    unit = align * sharding_degree
    total = (total + unit - 1) // unit * unit
    dev = parameters[0].device
    param_buffer = torch.zeros(total, dtype=dtype, device=dev)
    grad_buffer = None if release_grad else torch.zeros(total, dtype=torch.float32 if use_main_grad else dtype, device=dev)
    views = {}
    for p in parameters:
        off, padded = index[p.name]
        views[p.name] = ShardingGradView(p, param_buffer, grad_buffer, off, padded, sharding_degree, rank,
                                         use_main_grad, release_grad)
        if init_slice_param and slice_params is not None and p.name in slice_params:
            views[p.name].fill_slice_param(slice_params[p.name])
    return views, total, as_tensor(param_buffer), (as_tensor(grad_buffer) if grad_buffer is not None else None)
