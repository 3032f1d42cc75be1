"""The ``fleet`` singleton (python/paddle/distributed/fleet/fleet.py:218 ``init``, :674
``_init_hybrid_parallel_env``; fleet/model.py:33 ``distributed_model``; fleet/optimizer.py:24
``distributed_optimizer``)."""
from __future__ import annotations

import os
import time

import torch

from .. import collective as C
from ..parallel import ParallelEnv, init_parallel_env
from .base.distributed_strategy import DistributedStrategy
from .base.topology import CommunicateTopology, HybridCommunicateGroup, ParallelMode

_AXIS_OF = {"dp": "data", "pp": "pipe", "sharding": "sharding", "sep": "sep", "mp": "model"}


class Fleet:
    def __init__(self):
        self._is_collective = False
        self._user_defined_strategy = None
        self._hcg = None
        self._topology = None
        self._initialized = False

    # ------------------------------------------------------------------ init
    def init(self, role_maker=None, is_collective=False, strategy=None, log_level="INFO"):
        self._is_collective = is_collective or role_maker is None
        self._user_defined_strategy = strategy or DistributedStrategy()
        if not self._is_collective:
            raise NotImplementedError("parameter-server mode is not part of this framework")
        init_parallel_env()
        self._init_hybrid_parallel_env()
        self._initialized = True
        return self

    def _init_hybrid_parallel_env(self):
        hc = self._user_defined_strategy.hybrid_configs
        world = C.get_world_size()
        degrees = {"mp": hc["mp_degree"], "pp": hc["pp_degree"], "sharding": hc["sharding_degree"],
                   "sep": hc["sep_degree"], "dp": hc["dp_degree"]}
        other = degrees["mp"] * degrees["pp"] * degrees["sharding"] * degrees["sep"]
        if degrees["dp"] < 0:
            assert world % other == 0, f"world size {world} is not divisible by mp*pp*sharding*sep = {other}"
            degrees["dp"] = world // other
        hc.assign({"dp_degree": degrees["dp"]})
        order = list(hc["order"])
        names = [_AXIS_OF[o] for o in order]
        dims = [degrees[o] for o in order]
        self._topology = CommunicateTopology(names, dims)
        self._hcg = HybridCommunicateGroup(self._topology)
        if degrees["mp"] > 1:
            from .layers.mpu.random import model_parallel_random_seed
            seed = self._user_defined_strategy.tensor_parallel_configs["tensor_init_seed"]
            model_parallel_random_seed(None if seed == -1 else seed)

    # ------------------------------------------------------------------ info
    def get_hybrid_communicate_group(self):
        assert self._hcg is not None, "fleet.init must be called first"
        return self._hcg

    def get_hybrid_parallel_topology(self):
        return self._topology

    def is_first_worker(self):
        return C.get_rank() == 0

    def worker_index(self):
        return C.get_rank()

    def worker_num(self):
        return C.get_world_size()

    def node_num(self):
        return int(os.environ.get("PADDLE_NNODES", "1"))

    def local_rank(self):
        return int(os.environ.get("PADDLE_RANK_IN_NODE", os.environ.get("LOCAL_RANK", "0")))

    def local_device_ids(self):
        return [ParallelEnv().device_id]

    def world_device_ids(self):
        return list(range(C.get_world_size()))

    def is_worker(self):
        return True

    def is_server(self):
        return False

    def worker_endpoints(self, to_string=False):
        eps = ParallelEnv().trainer_endpoints
        return ",".join(eps) if to_string else eps

    def barrier_worker(self):
        C.barrier()

    def all_reduce(self, input, mode="sum"):
        """Reduce a Python number / array over all workers (``sum``, ``mean`` or ``max``); returns a numpy array, the
        input itself with a single worker (python/paddle/distributed/fleet/fleet.py ``all_reduce``)."""
        import numpy as np
        if mode not in ("sum", "mean", "max"):
            raise ValueError(f"mode should be sum, mean or max, got {mode!r}")
        arr = np.asarray(input)
        if not C.is_initialized() or C.get_world_size() == 1:
            return arr
        t = torch.as_tensor(arr.astype("float64") if arr.dtype.kind in "iu" and mode == "mean" else arr)
        on_gpu = (C._get_default_group().backend or "").lower() == "nccl"
        t = t.to(torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu"))
        C.all_reduce(t, C.ReduceOp.MAX if mode == "max" else C.ReduceOp.SUM)
        if mode == "mean":
            t = t / C.get_world_size()
        return t.cpu().numpy()

    def init_worker(self):
        pass

    def stop_worker(self):
        pass

    # ------------------------------------------------------------------ collective micro-benchmarks
    def _perf(self, fn, nbytes, iters, what, threshold):
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        for _ in range(2):
            fn()
        if dev == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        if dev == "cuda":
            torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) / iters * 1e3
        if threshold is not None and ms > threshold and C.get_rank() == 0:
            print(f"[Perf Warning] {what} of {nbytes} bytes took {ms:.3f} ms > threshold {threshold} ms")
        return ms

    def allreduce_perf(self, iteration, x, group, perf_size, perf_threshold_time, warmup=False):
        return self._perf(lambda: C.all_reduce(x, group=group), perf_size, iteration, "allreduce", perf_threshold_time)

    def broadcast_perf(self, iteration, x, group, perf_size, perf_threshold_time, warmup=False):
        return self._perf(lambda: C.broadcast(x, group.ranks[0], group), perf_size, iteration, "broadcast",
                          perf_threshold_time)

    def allgather_perf(self, iteration, x, group, perf_size, perf_threshold_time, warmup=False):
        out = torch.empty((group.nranks * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        return self._perf(lambda: C.all_gather(out, x, group), perf_size, iteration, "allgather", perf_threshold_time)

    def reduce_scatter_perf(self, iteration, x, group, perf_size, perf_threshold_time, warmup=False):
        out = torch.empty((x.shape[0] // group.nranks, *x.shape[1:]), dtype=x.dtype, device=x.device)
        return self._perf(lambda: C.reduce_scatter(out, x, group=group), perf_size, iteration, "reduce_scatter",
                          perf_threshold_time)

    def collective_perf(self, comm_type, round=50, size_and_time=None):
        size_and_time = size_and_time or {1 << 20: None, 1 << 26: None}
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        g = C._get_default_group()
        out = {}
        for nbytes, thr in size_and_time.items():
            n = max(nbytes // 4 // g.nranks * g.nranks, g.nranks)
            x = torch.zeros(n, dtype=torch.float32, device=dev)
            fn = {"allreduce": self.allreduce_perf, "broadcast": self.broadcast_perf, "allgather": self.allgather_perf,
                  "reduce_scatter": self.reduce_scatter_perf}[comm_type]
            out[nbytes] = fn(round, x, g, nbytes, thr)
        return out

    # ------------------------------------------------------------------ wrappers
    def distributed_model(self, model):
        """Pick the wrapper by parallel mode, precedence pp > mp > sep > sharding > dp
        (topology.py:292-328, fleet/model.py:143-186)."""
        hcg = self.get_hybrid_communicate_group()
        mode = hcg.get_parallel_mode()
        strategy = self._user_defined_strategy
        from . import meta_parallel as mp
        if mode == ParallelMode.PIPELINE_PARALLEL:
            from .meta_parallel.pipeline_parallel import PipelineParallel, PipelineParallelWithInterleave
            vpp = getattr(model, "get_num_virtual_stages", lambda: 1)()
            cfg = strategy.pipeline_configs
            mode = cfg.get("schedule_mode", "1F1B") if hasattr(cfg, "get") else "1F1B"
            # the schedules that exist only as generated step lists (zero bubble) run on the schedule executor
            cls = PipelineParallelWithInterleave if vpp > 1 or mode in ("ZBH1",) else PipelineParallel
            return cls(model, hcg, strategy=strategy)
        if mode == ParallelMode.TENSOR_PARALLEL:
            return mp.TensorParallel(model, hcg, strategy=strategy)
        if mode == ParallelMode.SEGMENT_PARALLEL:
            return mp.SegmentParallel(model, hcg, strategy=strategy)
        if mode == ParallelMode.SHARDING_PARALLEL:
            return mp.ShardingParallel(model, hcg, strategy=strategy)
        if hcg.get_data_parallel_world_size() > 1:
            from ..parallel import DataParallel
            return DataParallel(model, comm_buffer_size=strategy.fuse_grad_size_in_MB,
                                last_comm_buffer_size=strategy.last_comm_group_size_MB,
                                find_unused_parameters=strategy.find_unused_parameters,
                                group=hcg.get_data_parallel_group())
        return model

    def distributed_optimizer(self, optimizer, strategy=None):
        if strategy is not None:
            self._user_defined_strategy = strategy
        hcg = self.get_hybrid_communicate_group()
        if C.get_world_size() == 1:
            return optimizer
        from .meta_optimizers.dygraph_optimizer.hybrid_parallel_optimizer import HybridParallelOptimizer
        return HybridParallelOptimizer(optimizer, hcg, self._user_defined_strategy)

    def distributed_scaler(self, scaler):
        from .meta_optimizers.dygraph_optimizer.hybrid_parallel_gradscaler import HybridParallelGradScaler
        return HybridParallelGradScaler(scaler, self.get_hybrid_communicate_group())

    def state_dict(self):
        return {}

    def save_persistables(self, *a, **k):
        raise NotImplementedError("use paddle.save on the layer's state_dict")


fleet = Fleet()
