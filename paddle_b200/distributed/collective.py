"""Groups and collectives of ``paddle.distributed`` (python/paddle/distributed/collective.py,
communication/*.py, communication/stream/*.py).

One process per GPU.  The transport is a ``torch.distributed`` process group (NCCL on GPU, gloo on
CPU); this module supplies Paddle's object model on top: ``Group`` objects with ids and rank lists,
``ReduceOp``, collectives that return a ``task`` with ``wait()/is_completed()``, the ``sync_op`` /
``use_calc_stream`` issue modes of ``paddle.distributed.stream.*`` (communication/stream/all_reduce.py:38-55),
static argument checks (paddle/phi/core/distributed/check/static_check.cc:26-154) and optional dynamic
cross-rank checks (check/nccl_dynamic_check.cc:46-163) under ``FLAGS_enable_nccl_dynamic_check``.
"""
from __future__ import annotations

import datetime
import os
import pickle

import numpy as np
import torch
import torch.distributed as tdist

from .._core.tensor import as_tensor
from ..framework.flags import flag


class ReduceOp:
    SUM = 0
    MAX = 1
    MIN = 2
    PROD = 3
    AVG = 4


_TORCH_OP = {ReduceOp.SUM: tdist.ReduceOp.SUM, ReduceOp.MAX: tdist.ReduceOp.MAX, ReduceOp.MIN: tdist.ReduceOp.MIN,
             ReduceOp.PROD: tdist.ReduceOp.PRODUCT, ReduceOp.AVG: tdist.ReduceOp.AVG}


class Group:
    """python/paddle/distributed/communication/group.py ``Group``."""

    def __init__(self, rank_in_group, gid, ranks, pg=None, name=None):
        self._rank_in_group = rank_in_group
        self._world_size = len(ranks) if rank_in_group >= 0 else -1
        self._id = gid
        self._ranks = list(ranks)
        self._pg = pg
        self._name = name

    rank = property(lambda self: self._rank_in_group)
    ranks = property(lambda self: self._ranks)
    nranks = property(lambda self: len(self._ranks))
    world_size = property(lambda self: self._world_size)
    id = property(lambda self: self._id)
    name = property(lambda self: self._name)
    process_group = property(lambda self: self._pg)
    backend = property(lambda self: tdist.get_backend(self._pg) if self._pg is not None else None)

    def is_member(self):
        return self._rank_in_group >= 0 and self.nranks > 1 or self.nranks == 1 and self._rank_in_group >= 0

    def get_group_rank(self, rank):
        return self._ranks.index(rank) if rank in self._ranks else -1

    def __repr__(self):
        return f"rank: {self.rank}, nranks: {self.nranks}, id: {self.id}, ranks: {self._ranks}; name: {self._name}"


class _Task:
    """Completion handle of an asynchronous collective (ProcessGroup::Task in the reference)."""

    def __init__(self, work=None, post=None):
        self._work, self._post, self._done = work, post, work is None

    def wait(self, timeout=None):
        if self._work is not None:
            self._work.wait()
            self._work = None
        if self._post is not None:
            self._post()
            self._post = None
        self._done = True
        return True

    def is_completed(self):
        if self._done:
            return True
        if self._work is not None and self._work.is_completed():
            return True
        return False

    def synchronize(self):
        self.wait()


_group_map = {}
_default_group = None
_next_gid = [1]


def is_initialized():
    return _default_group is not None and tdist.is_initialized()


def is_available():
    return tdist.is_available()


def _set_default_group(g):
    global _default_group
    _default_group = g
    _group_map[0] = g


def _get_default_group():
    if _default_group is None:
        raise RuntimeError("Call paddle.distributed.init_parallel_env first to initialize the distributed environment.")
    return _default_group


def _get_global_group():
    return _get_default_group()


def get_rank(group=None):
    if group is not None:
        return group.rank
    if tdist.is_initialized():
        return tdist.get_rank()
    return int(os.environ.get("PADDLE_TRAINER_ID", os.environ.get("RANK", "0")))


def get_world_size(group=None):
    if group is not None:
        return group.nranks
    if tdist.is_initialized():
        return tdist.get_world_size()
    return int(os.environ.get("PADDLE_TRAINERS_NUM", os.environ.get("WORLD_SIZE", "1")))


def get_group(gid=0):
    return _group_map.get(gid)


def get_backend(group=None):
    g = group or _get_default_group()
    return g.backend.upper() if g.backend else None


def new_group(ranks=None, backend=None, timeout=datetime.timedelta(seconds=1800), nccl_comm_init_option=0):
    """Every rank of the job must call this (python/paddle/distributed/collective.py:195)."""
    default = _get_default_group()
    world = default.nranks
    ranks = sorted(ranks) if ranks is not None else list(range(world))
    gid = _next_gid[0]
    _next_gid[0] += 1
    me = tdist.get_rank()
    pg = tdist.new_group(ranks=ranks, timeout=timeout, backend=backend.lower() if backend else None)
    rank_in = ranks.index(me) if me in ranks else -1
    g = Group(rank_in, gid, ranks, pg if rank_in >= 0 else None, name=f"_default_pg{gid}")
    _group_map[gid] = g
    return g


def destroy_process_group(group=None):
    global _default_group
    if group is None or group is _default_group:
        if tdist.is_initialized():
            tdist.destroy_process_group()
        _group_map.clear()
        _default_group = None
    else:
        if group.process_group is not None:
            tdist.destroy_process_group(group.process_group)
        _group_map.pop(group.id, None)


# ------------------------------------------------------------------------------------- checks
def _static_check(tensor, group, what, root=None):
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{what}: expected a Tensor, got {type(tensor)}")
    if root is not None and not (0 <= root < group.nranks):
        raise ValueError(f"{what}: rank {root} is out of range for a group of {group.nranks}")
    if tdist.get_backend(group.process_group) == "nccl" and not tensor.is_cuda:
        raise ValueError(f"{what}: NCCL collectives need GPU tensors")


def _dynamic_check(tensor, group, what):
    """Compare (dtype, shape) of every rank with rank 0 of the group; raises on mismatch."""
    if not flag("enable_nccl_dynamic_check"):
        return
    meta = torch.tensor([hash(str(tensor.dtype)) % (1 << 31), tensor.dim(), *tensor.shape] + [0] * (8 - tensor.dim()),
                        dtype=torch.int64, device=tensor.device)
    ref = meta.clone()
    tdist.broadcast(ref, group.ranks[0], group=group.process_group)
    if not torch.equal(ref, meta):
        raise RuntimeError(f"{what}: dtype/shape differs from rank {group.ranks[0]} of the group: "
                           f"{meta.tolist()} vs {ref.tolist()}")


def _grp(group):
    g = group if group is not None else _get_default_group()
    return g


def _finish(work, sync_op, use_calc_stream=False, post=None):
    if sync_op or use_calc_stream or work is None:
        if work is not None:
            work.wait()
        if post is not None:
            post()
        return _Task(None)
    return _Task(work, post)


def _plain(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) and type(t) is not torch.Tensor else t


# ------------------------------------------------------------------------------------- collectives
def all_reduce(tensor, op=ReduceOp.SUM, group=None, sync_op=True, use_calc_stream=False):
    g = _grp(group)
    if g.nranks == 1 or not g.is_member():
        return _Task(None)
    _static_check(tensor, g, "all_reduce")
    _dynamic_check(tensor, g, "all_reduce")
    top = _TORCH_OP[op]
    if op == ReduceOp.AVG and tdist.get_backend(g.process_group) == "gloo":
        w = tdist.all_reduce(_plain(tensor), tdist.ReduceOp.SUM, group=g.process_group, async_op=True)
        return _finish(w, sync_op, use_calc_stream, post=lambda: tensor.div_(g.nranks))
    w = tdist.all_reduce(_plain(tensor), top, group=g.process_group, async_op=True)
    return _finish(w, sync_op, use_calc_stream)


def broadcast(tensor, src=0, group=None, sync_op=True, use_calc_stream=False):
    g = _grp(group)
    if g.nranks == 1 or not g.is_member():
        return _Task(None)
    _static_check(tensor, g, "broadcast")
    w = tdist.broadcast(_plain(tensor), src, group=g.process_group, async_op=True)
    return _finish(w, sync_op, use_calc_stream)


def reduce(tensor, dst=0, op=ReduceOp.SUM, group=None, sync_op=True, use_calc_stream=False):
    g = _grp(group)
    if g.nranks == 1 or not g.is_member():
        return _Task(None)
    _static_check(tensor, g, "reduce")
    if op == ReduceOp.AVG:
        w = tdist.reduce(_plain(tensor), dst, tdist.ReduceOp.SUM, group=g.process_group, async_op=True)
        return _finish(w, sync_op, use_calc_stream,
                       post=(lambda: tensor.div_(g.nranks)) if tdist.get_rank() == dst else None)
    w = tdist.reduce(_plain(tensor), dst, _TORCH_OP[op], group=g.process_group, async_op=True)
    return _finish(w, sync_op, use_calc_stream)


def all_gather(tensor_list, tensor, group=None, sync_op=True, use_calc_stream=False):
    """``tensor_list`` may be a list (filled with the per-rank tensors) or a single tensor that
    receives the concatenation along axis 0 (``all_gather_into_tensor`` form)."""
    g = _grp(group)
    if isinstance(tensor_list, torch.Tensor):
        if g.nranks == 1:
            tensor_list.copy_(tensor.reshape(tensor_list.shape))
            return _Task(None)
        w = tdist.all_gather_into_tensor(_plain(tensor_list), _plain(tensor.contiguous()), group=g.process_group,
                                         async_op=True)
        return _finish(w, sync_op, use_calc_stream)
    if g.nranks == 1:
        tensor_list.clear()
        tensor_list.append(tensor)
        return _Task(None)
    _static_check(tensor, g, "all_gather")
    outs = [torch.empty_like(_plain(tensor)) for _ in range(g.nranks)]
    w = tdist.all_gather(outs, _plain(tensor.contiguous()), group=g.process_group, async_op=True)

    def post():
        tensor_list.clear()
        tensor_list.extend(as_tensor(o) for o in outs)
    return _finish(w, sync_op, use_calc_stream, post=post)


def all_gather_into_tensor(out_tensor, tensor, group=None, sync_op=True, use_calc_stream=False):
    return all_gather(out_tensor, tensor, group, sync_op, use_calc_stream)


def reduce_scatter(tensor, tensor_list, op=ReduceOp.SUM, group=None, sync_op=True, use_calc_stream=False):
    """``tensor_list``: list of per-rank inputs or one tensor whose axis 0 is split across ranks."""
    g = _grp(group)
    if g.nranks == 1:
        src = tensor_list if isinstance(tensor_list, torch.Tensor) else tensor_list[0]
        tensor.copy_(src.reshape(tensor.shape))
        return _Task(None)
    src = tensor_list if isinstance(tensor_list, torch.Tensor) else torch.cat([_plain(t) for t in tensor_list], 0)
    if tdist.get_backend(g.process_group) == "gloo":   # gloo has no reduce_scatter: all_reduce + slice
        full = _plain(src).clone()
        w = tdist.all_reduce(full, _TORCH_OP[ReduceOp.SUM if op == ReduceOp.AVG else op], group=g.process_group,
                             async_op=True)

        def post():
            n = full.shape[0] // g.nranks
            part = full[g.rank * n:(g.rank + 1) * n]
            tensor.copy_((part / g.nranks if op == ReduceOp.AVG else part).reshape(tensor.shape))
        return _finish(w, sync_op, use_calc_stream, post=post)
    w = tdist.reduce_scatter_tensor(_plain(tensor), _plain(src.contiguous()), _TORCH_OP[op], group=g.process_group,
                                    async_op=True)
    return _finish(w, sync_op, use_calc_stream)


def alltoall(out_tensor_list, in_tensor_list, group=None, sync_op=True, use_calc_stream=False):
    """Tensor i of ``in_tensor_list`` goes to rank i; ``out_tensor_list`` receives one tensor per rank (argument order of
    python/paddle/distributed/communication/all_to_all.py:26: outputs first)."""
    return _alltoall_io(in_tensor_list, out_tensor_list, group, sync_op, use_calc_stream)


def _alltoall_io(in_tensor_list, out_tensor_list, group=None, sync_op=True, use_calc_stream=False):
    g = _grp(group)
    if g.nranks == 1:
        out_tensor_list.clear()
        out_tensor_list.extend(in_tensor_list)
        return _Task(None)
    ins = [_plain(t.contiguous()) for t in in_tensor_list]
    outs = [torch.empty_like(t) for t in ins] if not out_tensor_list else [_plain(t) for t in out_tensor_list]
    if tdist.get_backend(g.process_group) == "gloo":
        reqs = []
        for i in range(g.nranks):
            if i == g.rank:
                outs[i].copy_(ins[i])
                continue
            reqs.append(tdist.isend(ins[i], g.ranks[i], group=g.process_group))
            reqs.append(tdist.irecv(outs[i], g.ranks[i], group=g.process_group))
        for r in reqs:
            r.wait()
        w = None
    else:
        w = tdist.all_to_all(outs, ins, group=g.process_group, async_op=True)

    def post():
        if not out_tensor_list:
            out_tensor_list.extend(as_tensor(o) for o in outs)
    return _finish(w, sync_op, use_calc_stream, post=post) if w is not None else (post() or _Task(None))


all_to_all = alltoall


def alltoall_single(out_tensor, in_tensor, in_split_sizes=None, out_split_sizes=None, group=None, sync_op=True,
                    use_calc_stream=False):
    """Rows of ``in_tensor`` are split over the ranks (evenly or by ``in_split_sizes``); ``out_tensor`` receives the
    pieces in rank order (python/paddle/distributed/communication/all_to_all.py:78: output first)."""
    return _alltoall_single_io(in_tensor, out_tensor, in_split_sizes, out_split_sizes, group, sync_op, use_calc_stream)


def _alltoall_single_io(in_tensor, out_tensor, in_split_sizes=None, out_split_sizes=None, group=None, sync_op=True,
                        use_calc_stream=False):
    g = _grp(group)
    if g.nranks == 1:
        out_tensor.copy_(in_tensor)
        return _Task(None)
    if tdist.get_backend(g.process_group) == "gloo":
        n = g.nranks
        ins = list(torch.split(_plain(in_tensor), in_split_sizes or in_tensor.shape[0] // n, 0))
        outs = list(torch.split(_plain(out_tensor), out_split_sizes or out_tensor.shape[0] // n, 0))
        return _alltoall_io(ins, outs, group, sync_op, use_calc_stream)
    w = tdist.all_to_all_single(_plain(out_tensor), _plain(in_tensor.contiguous()), out_split_sizes, in_split_sizes,
                                group=g.process_group, async_op=True)
    return _finish(w, sync_op, use_calc_stream)


def scatter(tensor, tensor_list=None, src=0, group=None, sync_op=True, use_calc_stream=False):
    g = _grp(group)
    if g.nranks == 1:
        tensor.copy_(tensor_list[0])
        return _Task(None)
    me = tdist.get_rank()
    lst = [_plain(t.contiguous()) for t in tensor_list] if me == src and tensor_list else None
    if tdist.get_backend(g.process_group) == "nccl":
        # NCCL scatter through point-to-point, as ProcessGroupNCCL::Scatter does (process_group_nccl.cc:499)
        if me == src:
            reqs = [tdist.isend(lst[i], r, group=g.process_group) for i, r in enumerate(g.ranks) if r != me]
            tensor.copy_(lst[g.ranks.index(me)])
            for r in reqs:
                r.wait()
        else:
            tdist.recv(_plain(tensor), src, group=g.process_group)
        return _Task(None)
    w = tdist.scatter(_plain(tensor), lst, src, group=g.process_group, async_op=True)
    return _finish(w, sync_op, use_calc_stream)


def gather(tensor, gather_list=None, dst=0, group=None, sync_op=True, use_calc_stream=False):
    g = _grp(group)
    if g.nranks == 1:
        if gather_list is not None:
            gather_list.clear()
            gather_list.append(tensor)
        return _Task(None)
    tmp = []
    all_gather(tmp, tensor, group)
    if tdist.get_rank() == dst and gather_list is not None:
        gather_list.clear()
        gather_list.extend(tmp)
    return _Task(None)


def send(tensor, dst=0, group=None, sync_op=True, use_calc_stream=False):
    g = _grp(group)
    _static_check(tensor, g, "send")
    w = tdist.isend(_plain(tensor.contiguous()), dst, group=g.process_group)
    return _finish(w, sync_op, use_calc_stream)


def recv(tensor, src=0, group=None, sync_op=True, use_calc_stream=False):
    g = _grp(group)
    _static_check(tensor, g, "recv")
    w = tdist.irecv(_plain(tensor), src, group=g.process_group)
    return _finish(w, sync_op, use_calc_stream)


def isend(tensor, dst, group=None):
    return send(tensor, dst, group, sync_op=False)


def irecv(tensor, src=None, group=None):
    return recv(tensor, src, group, sync_op=False)


class P2POp:
    def __init__(self, op, tensor, peer, group=None):
        if op not in (isend, irecv, send, recv):
            raise RuntimeError("op must be paddle.distributed.isend or irecv")
        self.op, self.tensor, self.peer, self.group = op, tensor, peer, group


def batch_isend_irecv(p2p_op_list):
    """Issue a batch of sends/receives as one group (ncclGroupStart/End in the reference,
    python/paddle/distributed/communication/batch_isend_irecv.py)."""
    if not p2p_op_list:
        return []
    g = _grp(p2p_op_list[0].group)
    ops = [tdist.P2POp(tdist.isend if o.op in (isend, send) else tdist.irecv, _plain(o.tensor), o.peer,
                       group=g.process_group) for o in p2p_op_list]
    works = tdist.batch_isend_irecv(ops)
    return [_Task(w) for w in works]


def barrier(group=None):
    g = _grp(group)
    if g.nranks == 1:
        return
    if tdist.get_backend(g.process_group) == "nccl":
        tdist.barrier(group=g.process_group, device_ids=[torch.cuda.current_device()])
    else:
        tdist.barrier(group=g.process_group)


def wait(tensor, group=None, use_calc_stream=True):
    if tensor.is_cuda:
        torch.cuda.current_stream().synchronize() if not use_calc_stream else None


# ------------------------------------------------------------------------------------- object collectives
def _obj_to_tensor(obj, device):
    data = np.frombuffer(pickle.dumps(obj), dtype=np.uint8).copy()
    return torch.from_numpy(data).to(device), data.size


def _dev(g):
    return torch.device("cuda", torch.cuda.current_device()) if tdist.get_backend(g.process_group) == "nccl" \
        else torch.device("cpu")


def all_gather_object(object_list, obj, group=None):
    g = _grp(group)
    if g.nranks == 1:
        object_list.clear()
        object_list.append(obj)
        return
    out = [None] * g.nranks
    tdist.all_gather_object(out, obj, group=g.process_group)
    object_list.clear()
    object_list.extend(out)


def broadcast_object_list(object_list, src=0, group=None):
    g = _grp(group)
    if g.nranks == 1:
        return
    tdist.broadcast_object_list(object_list, src, group=g.process_group)


def scatter_object_list(out_object_list, in_object_list=None, src=0, group=None):
    g = _grp(group)
    if g.nranks == 1:
        out_object_list.clear()
        out_object_list.append(in_object_list[0])
        return
    tmp = [None]
    tdist.scatter_object_list(tmp, in_object_list if tdist.get_rank() == src else None, src, group=g.process_group)
    out_object_list.clear()
    out_object_list.extend(tmp)


def gather_object(obj, object_gather_list=None, dst=0, group=None):
    tmp = []
    all_gather_object(tmp, obj, group)
    if tdist.get_rank() == dst and object_gather_list is not None:
        object_gather_list.clear()
        object_gather_list.extend(tmp)
