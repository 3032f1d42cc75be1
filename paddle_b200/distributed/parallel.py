"""``init_parallel_env``, ``ParallelEnv`` and ``DataParallel`` (python/paddle/distributed/parallel.py:978,
:219).  Rank / world size / endpoints come from the launcher's ``PADDLE_*`` variables
(parallel.py:1104-1133) or, when launched by ``torch.distributed.run``, from ``RANK``/``WORLD_SIZE``/
``MASTER_ADDR``/``MASTER_PORT``.  Rendezvous goes through a TCP store served by rank 0."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as tdist

from .._core import dtype as _dt
from ..nn.layer.layers import Layer
from . import collective as C


class ParallelEnv:
    def __init__(self):
        e = os.environ
        self._rank = int(e.get("PADDLE_TRAINER_ID", e.get("RANK", "0")))
        self._world_size = int(e.get("PADDLE_TRAINERS_NUM", e.get("WORLD_SIZE", "1")))
        self._device_id = int(e.get("FLAGS_selected_gpus", e.get("LOCAL_RANK", "0")).split(",")[0])
        eps = e.get("PADDLE_TRAINER_ENDPOINTS", "")
        self._trainer_endpoints = eps.split(",") if eps else []
        self._current_endpoint = e.get("PADDLE_CURRENT_ENDPOINT", "")
        self._nrings = int(e.get("FLAGS_nccl_nrings", "1"))
        self.pg_timeout = int(e.get("PADDLE_PG_TIMEOUT", "1800000"))

    rank = property(lambda self: self._rank)
    local_rank = property(lambda self: self._rank)
    world_size = property(lambda self: self._world_size)
    nranks = property(lambda self: self._world_size)
    device_id = property(lambda self: self._device_id)
    dev_id = property(lambda self: self._device_id)
    current_endpoint = property(lambda self: self._current_endpoint)
    trainer_endpoints = property(lambda self: self._trainer_endpoints)
    nrings = property(lambda self: self._nrings)


def _master_from_env():
    e = os.environ
    if "PADDLE_MASTER" in e:
        host, port = e["PADDLE_MASTER"].rsplit(":", 1)
        return host, int(port)
    eps = e.get("PADDLE_TRAINER_ENDPOINTS", "")
    if eps:
        host, port = eps.split(",")[0].rsplit(":", 1)
        return host, int(port)
    return e.get("MASTER_ADDR", "127.0.0.1"), int(e.get("MASTER_PORT", "29500"))


def init_parallel_env(backend=None):
    """Create the default group.  Backend: NCCL when a GPU is present, otherwise gloo;
    ``PADDLE_DISTRI_BACKEND=gloo`` forces the CPU backend."""
    if C.is_initialized():
        return C._get_default_group()
    env = ParallelEnv()
    backend = (backend or os.environ.get("PADDLE_DISTRI_BACKEND") or
               ("nccl" if torch.cuda.is_available() else "gloo")).lower()
    if backend in ("auto",):
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        dev = env.device_id if torch.cuda.device_count() > env.device_id else 0
        torch.cuda.set_device(dev)
        _dt.set_device(f"gpu:{dev}")
    if not tdist.is_initialized():
        host, port = _master_from_env()
        timeout = datetime.timedelta(milliseconds=env.pg_timeout)
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        tdist.init_process_group(backend, init_method=f"tcp://{host}:{port}", rank=env.rank,
                                 world_size=env.world_size, timeout=timeout, **kw)
    world = tdist.get_world_size()
    g = C.Group(tdist.get_rank(), 0, list(range(world)), tdist.group.WORLD, name="_default_pg")
    C._set_default_group(g)
    if backend == "gloo":
        # gloo keeps worker threads per group; leaving the interpreter with them alive ends some runs with
        # "terminate called without an active exception", so the groups are taken down at exit
        import atexit

        def _shutdown():
            try:
                if tdist.is_initialized():
                    tdist.destroy_process_group()
            except Exception:  # noqa: BLE001 - never turn a clean exit into a failure
                pass
        atexit.register(_shutdown)
    from ..framework.flags import flag
    if flag("enable_async_trace"):
        from . import watchdog
        if not watchdog.enabled():
            watchdog.start(timeout_s=env.pg_timeout / 1000.0)
    return g


def get_rank(group=None):
    return C.get_rank(group)


def get_world_size(group=None):
    return C.get_world_size(group)


def sync_params_buffers(model, comm_group=None, src_rank=0, is_model_parallel=False, fuse_params=True):
    """Broadcast parameters and buffers from ``src_rank`` (parallel.py ``sync_params_buffers``)."""
    with torch.no_grad():
        for t in list(model.parameters()) + list(model.buffers()):
            if is_model_parallel and getattr(t, "is_distributed", False):
                continue
            C.broadcast(t.data if hasattr(t, "data") else t, src_rank, comm_group)


class DataParallel(Layer):
    """Bucketed gradient all-reduce overlapped with backward (EagerReducer,
    paddle/fluid/distributed/collective/reducer.cc:482): parameters are grouped into buckets of
    ``comm_buffer_size`` MB in reverse order; when every gradient of a bucket has been accumulated the
    flat bucket is all-reduced asynchronously; ``no_sync()`` suspends communication for accumulation."""

    def __init__(self, layers, strategy=None, comm_buffer_size=25, last_comm_buffer_size=1, find_unused_parameters=False,
                 group=None):
        super().__init__()
        self._layers = layers
        self.group = group
        self.find_unused_parameters = find_unused_parameters
        self._sync = True
        self._comm_buffer_bytes = int(comm_buffer_size * 1024 * 1024)
        self._last_comm_buffer_bytes = int(last_comm_buffer_size * 1024 * 1024)
        self._nranks = C.get_world_size(group) if C.is_initialized() else 1
        self._pending = []
        if self._nranks > 1:
            sync_params_buffers(layers, group, (group.ranks[0] if group is not None else 0))
            self._build_buckets()

    def _build_buckets(self):
        from .reducer import assign_group_by_size
        params = [p for p in self._layers.parameters() if p.requires_grad]
        self._params = params
        idx_groups = assign_group_by_size(params, [self._last_comm_buffer_bytes, self._comm_buffer_bytes])
        self._buckets = []
        self._param2bucket = {}
        for bi, idxs in enumerate(idx_groups):
            b = {"params": [params[i] for i in idxs], "ready": 0, "flat": None}
            self._buckets.append(b)
            for i in idxs:
                self._param2bucket[id(params[i])] = bi
        self._index = {id(p): i for i, p in enumerate(params)}
        bucket_of = [self._param2bucket[id(p)] for p in params]
        self._native = None
        try:
            import ctypes

            from ..ops import _lib
            rt = _lib.runtime()
            rt.pd_reducer_create.restype = ctypes.c_void_p
            arr = (ctypes.c_int * len(bucket_of))(*bucket_of)
            h = rt.pd_reducer_create(arr, len(bucket_of), len(self._buckets))
            if h:
                self._native = (rt, ctypes.c_void_p(h))
        except Exception:  # noqa: BLE001 - without the native runtime the same counters are kept in Python
            self._native = None
        self._seen = set()
        self._in_backward = False
        for p in params:
            p.register_post_accumulate_grad_hook(self._make_hook())

    def _mark_ready(self, p):
        """-> (bucket index | -1 incomplete | -2 duplicate, first arrival of this backward)."""
        if self._native is not None:
            import ctypes
            rt, h = self._native
            first = ctypes.c_int(0)
            return rt.pd_reducer_mark_ready(h, self._index[id(p)], ctypes.byref(first)), bool(first.value)
        first = not self._in_backward
        self._in_backward = True
        if id(p) in self._seen:
            return -2, first
        self._seen.add(id(p))
        bi = self._param2bucket[id(p)]
        b = self._buckets[bi]
        b["ready"] += 1
        if b["ready"] == len(b["params"]):
            b["launched"] = True
            return bi, first
        return -1, first

    def _unfinished(self):
        """Buckets that did not complete in the backward pass that just ended; resets the counters."""
        if self._native is not None:
            import ctypes
            rt, h = self._native
            out = (ctypes.c_int * len(self._buckets))()
            n = rt.pd_reducer_finish(h, out, len(self._buckets))
            return [out[i] for i in range(n)]
        left = [i for i, b in enumerate(self._buckets) if not b.get("launched")]
        for b in self._buckets:
            b["ready"], b["launched"] = 0, False
        self._seen.clear()
        self._in_backward = False
        return left

    def _make_hook(self):
        def hook(p):
            if not self._sync:
                return
            bi, first = self._mark_ready(p)
            if first:
                # the end-of-backward work is queued by the FIRST gradient of the pass, not by the first complete bucket:
                # a pass in which no bucket completes (an unused parameter in a one-bucket model) must still be finished,
                # or its stale counts would fire a bucket in the middle of the next pass
                torch.autograd.Variable._execution_engine.queue_callback(self._finalize)
            if bi == -2:
                raise RuntimeError(f"gradient of {getattr(p, 'name', 'a parameter')} was produced twice in one backward "
                                   "pass; wrap the extra passes in no_sync()")
            if bi >= 0:
                self._launch(self._buckets[bi])
        return hook

    def _launch(self, b):
        grads = [torch.Tensor.grad.__get__(p) for p in b["params"]]
        flat = torch.cat([g.reshape(-1) for g in grads])
        flat.div_(self._nranks)
        task = C.all_reduce(flat, group=self.group, sync_op=False)
        self._pending.append((task, flat, grads))

    def _finalize(self):
        for task, flat, grads in self._pending:
            task.wait()
            off = 0
            for g in grads:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g))
                off += n
        self._pending.clear()
        left = self._unfinished()
        if not left:
            return
        if not self.find_unused_parameters:
            names = [getattr(p, "name", "?") for bi in left for p in self._buckets[bi]["params"]
                     if torch.Tensor.grad.__get__(p) is None]
            raise RuntimeError(
                "some parameters received no gradient in this backward pass, so their buckets were never reduced "
                f"({', '.join(names[:8])}{' ...' if len(names) > 8 else ''}).  Construct DataParallel with "
                "find_unused_parameters=True if parts of the model are skipped on purpose.")
        # parameters without a gradient this step take part with zeros so that every rank issues the same collectives
        for bi in left:
            b = self._buckets[bi]
            for p in b["params"]:
                if torch.Tensor.grad.__get__(p) is None:
                    p.grad = torch.zeros_like(p)
            grads = [torch.Tensor.grad.__get__(p) for p in b["params"]]
            flat = torch.cat([g.reshape(-1) for g in grads]).div_(self._nranks)
            C.all_reduce(flat, group=self.group)
            off = 0
            for g in grads:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()

    def no_sync(self):
        dp = self

        class _Ctx:
            def __enter__(self_):
                self_.prev = dp._sync
                dp._sync = False

            def __exit__(self_, *a):
                dp._sync = self_.prev
        return _Ctx()

    def forward(self, *inputs, **kwargs):
        return self._layers(*inputs, **kwargs)

    def state_dict(self, *a, **k):
        return self._layers.state_dict(*a, **k)

    def set_state_dict(self, *a, **k):
        return self._layers.set_state_dict(*a, **k)

    set_dict = load_dict = set_state_dict

    def scale_loss(self, loss):
        return loss

    def apply_collective_grads(self):
        pass


_gloo_group = None


def gloo_init_parallel_env(rank_id, rank_num, server_endpoint):
    """CPU-only process group over gloo with the store on ``server_endpoint`` (python/paddle/distributed/parallel.py
    ``gloo_init_parallel_env``); used for host-side barriers and small collectives before any GPU context exists."""
    global _gloo_group
    import datetime

    import torch.distributed as tdist
    ip, port = server_endpoint.rsplit(":", 1)
    store = tdist.TCPStore(ip, int(port), rank_num, rank_id == 0, timeout=datetime.timedelta(seconds=300))
    if tdist.is_initialized():
        _gloo_group = tdist.new_group(backend="gloo")
    else:
        tdist.init_process_group("gloo", store=store, rank=rank_id, world_size=rank_num)
        _gloo_group = tdist.group.WORLD


def gloo_barrier():
    import torch.distributed as tdist
    if _gloo_group is None:
        raise RuntimeError("call gloo_init_parallel_env first")
    tdist.barrier(group=_gloo_group)


def gloo_release():
    global _gloo_group
    import torch.distributed as tdist
    if _gloo_group is not None and _gloo_group is tdist.group.WORLD and tdist.is_initialized():
        tdist.destroy_process_group()
    _gloo_group = None
