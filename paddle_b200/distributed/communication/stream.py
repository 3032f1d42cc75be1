"""``paddle.distributed.stream.*``: collectives with explicit issue mode
(python/paddle/distributed/communication/stream/*.py:37-74).  ``sync_op=False`` returns a task to wait on;
``use_calc_stream=True`` (only with ``sync_op=True``) issues on the compute stream without a host wait."""
from __future__ import annotations

from .. import collective as C


def _check(sync_op, use_calc_stream):
    if use_calc_stream and not sync_op:
        raise RuntimeError("use_calc_stream can only be true in sync op behavior.")


def all_reduce(tensor, op=C.ReduceOp.SUM, group=None, sync_op=True, use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    return C.all_reduce(tensor, op, group, sync_op, use_calc_stream)


def all_gather(tensor_or_tensor_list, tensor, group=None, sync_op=True, use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    return C.all_gather(tensor_or_tensor_list, tensor, group, sync_op, use_calc_stream)


def reduce_scatter(tensor, tensor_or_tensor_list, op=C.ReduceOp.SUM, group=None, sync_op=True, use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    return C.reduce_scatter(tensor, tensor_or_tensor_list, op, group, sync_op, use_calc_stream)


def broadcast(tensor, src=0, group=None, sync_op=True, use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    return C.broadcast(tensor, src, group, sync_op, use_calc_stream)


def reduce(tensor, dst=0, op=C.ReduceOp.SUM, group=None, sync_op=True, use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    return C.reduce(tensor, dst, op, group, sync_op, use_calc_stream)


def alltoall(out_tensor_or_tensor_list, in_tensor_or_tensor_list, group=None, sync_op=True, use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    import torch
    if isinstance(in_tensor_or_tensor_list, torch.Tensor):
        return C._alltoall_single_io(in_tensor_or_tensor_list, out_tensor_or_tensor_list, None, None, group, sync_op,
                                 use_calc_stream)
    return C._alltoall_io(in_tensor_or_tensor_list, out_tensor_or_tensor_list, group, sync_op, use_calc_stream)


def alltoall_single(out_tensor, in_tensor, out_split_sizes=None, in_split_sizes=None, group=None, sync_op=True,
                    use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    return C._alltoall_single_io(in_tensor, out_tensor, in_split_sizes, out_split_sizes, group, sync_op, use_calc_stream)


def scatter(tensor, tensor_or_tensor_list=None, src=0, group=None, sync_op=True, use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    import torch
    lst = tensor_or_tensor_list
    if isinstance(lst, torch.Tensor):
        n = C.get_world_size(group)
        lst = list(lst.chunk(n, 0))
    return C.scatter(tensor, lst, src, group, sync_op, use_calc_stream)


def gather(tensor, gather_list=None, dst=0, group=None, sync_op=True, use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    return C.gather(tensor, gather_list, dst, group, sync_op, use_calc_stream)


def send(tensor, dst=0, group=None, sync_op=True, use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    return C.send(tensor, dst, group, sync_op, use_calc_stream)


def recv(tensor, src=0, group=None, sync_op=True, use_calc_stream=False):
    _check(sync_op, use_calc_stream)
    return C.recv(tensor, src, group, sync_op, use_calc_stream)
