"""Cost classes of the planner (python/paddle/distributed/auto_parallel/static/cost/base_cost.py): a ``Cost`` is
(time, memory, flops); ``CommContext`` turns the cluster description into start-up latency (alpha) and seconds per
byte (beta) of a collective over a given group of ranks; ``CommOpCost`` / ``CompOpCost`` are the bases of the
per-operator classes, which register themselves by operator type.  Times are seconds, sizes bytes."""
from __future__ import annotations

import math

COMM_OP_TYPE = ["send_v2", "recv_v2", "c_broadcast", "c_allgather", "c_allreduce_sum", "c_reducescatter", "all_to_all",
                "c_identity", "all_gather", "all_reduce", "reduce_scatter", "broadcast", "send", "recv"]
NON_COMP_TYPE = ["while", "conditional_block", *COMM_OP_TYPE]
_g_op_cost_factory = {}


def register_op_cost(cls):
    _g_op_cost_factory[cls.OP_TYPE] = cls
    for alias in getattr(cls, "ALIASES", ()):
        _g_op_cost_factory[alias] = cls
    return cls


class Cost:
    def __init__(self, time=0.0, memory=0, flops=0):
        self.time, self.memory, self.flops = float(time), int(memory), int(flops)

    def __add__(self, rhs):
        return Cost(self.time + rhs.time, self.memory + rhs.memory, self.flops + rhs.flops)

    def __sub__(self, rhs):
        return Cost(self.time - rhs.time, self.memory - rhs.memory, self.flops - rhs.flops)

    def __repr__(self):
        return f"Cost(time={self.time * 1e3:.4f} ms, memory={self.memory / 2 ** 20:.1f} MiB, flops={self.flops:.3e})"


class CommContext:
    """Alpha / beta of collectives on a cluster.  Inside a machine whose accelerators sit behind a switch, the rate a
    collective reaches grows with the number of ranks that take part (measured on an 8-GPU NVSwitch node: about half of
    the 8-rank bus bandwidth between two GPUs, three quarters among four); across machines the slowest link of the
    ring decides."""
    _instance = None
    _has_instance = False
    _SWITCH_SCALE = {2: 0.51, 4: 0.76, 8: 1.0}
    _BUS_FRACTION = 0.935          # 8-rank all-reduce bus bandwidth over the device-to-device copy rate, as measured

    def __new__(cls, cluster=None):
        if cls._instance is None or (cluster is not None and cluster is not cls._instance.cluster):
            cls._instance = super().__new__(cls)
            cls._instance._init(cluster)
            cls._has_instance = True
        return cls._instance

    def _init(self, cluster):
        if cluster is None:
            from ..cluster import get_default_cluster
            cluster = get_default_cluster()
        self.cluster = cluster
        al = cluster.alpha_latency
        self.base_ring = (al.base_ring if al and al.base_ring is not None else 8.4) * 1e-6
        self.base_tree = (al.base_tree if al and al.base_tree is not None else 0.0) * 1e-6
        self.intra_ring = (al.intra_ring if al and al.intra_ring is not None else 8.0) * 1e-6
        self.inter_ring = (al.inter_ring if al and al.inter_ring is not None else 9.6) * 1e-6
        self.switch = (al.switch if al and al.switch is not None else 10.0) * 1e-6
        self.beta, self.hops = {}, {}

    @classmethod
    def reset(cls):
        cls._instance, cls._has_instance = None, False

    def get_alpha(self, ranks, kind="ring"):
        if len(ranks) <= 1:
            return 0.0
        cross = self.cluster.cross_machine(ranks)
        return self.base_ring + (self.inter_ring + self.switch if cross else self.intra_ring)

    def get_beta(self, ranks):
        """Seconds per byte of payload for a collective over ``ranks``."""
        key = tuple(sorted(ranks))
        if key in self.beta:
            return self.beta[key]
        if len(key) <= 1:
            return 0.0
        worst = max(self.cluster.get_beta(a, b) for a, b in zip(key, key[1:] + key[:1]) if a != b)
        if not self.cluster.cross_machine(key):
            n = len(key)
            sc = self._SWITCH_SCALE
            if n in sc:
                f = sc[n]
            else:
                lo, hi = max(k for k in sc if k <= n), min((k for k in sc if k >= n), default=8)
                f = sc[lo] if lo == hi else sc[lo] + (math.log2(n) - math.log2(lo)) / (math.log2(hi) - math.log2(lo)) * (sc[hi] - sc[lo])
            worst = worst / (f * self._BUS_FRACTION)
        self.beta[key] = worst
        return worst


def build_comm_desc(op_type, group_ranks, dtype, shape, attrs=None):
    return {"op": op_type, "group_ranks": list(group_ranks), "inputs": {"X": [(dtype, list(shape))]}, "attrs": attrs or {}}


def _itemsize(dtype):
    import torch
    if isinstance(dtype, torch.dtype):
        return dtype.itemsize
    return {"float16": 2, "bfloat16": 2, "float32": 4, "float64": 8, "int32": 4, "int64": 8, "int8": 1, "uint8": 1, "bool": 1}.get(str(dtype).split(".")[-1], 4)


class OpCost:
    OP_TYPE = "op"

    def __init__(self, op=None, op_desc=None):
        self.op, self.op_desc = op, op_desc
        self._cost = None

    @property
    def time(self):
        return self.cost.time

    @property
    def memory(self):
        return self.cost.memory

    @property
    def flops(self):
        return self.cost.flops

    @property
    def cost(self):
        if self._cost is None:
            self._cost = Cost(self.calc_time(), self.calc_memory(), self.calc_flops())
        return self._cost

    def calc_time(self):
        return 0.0

    def calc_memory(self):
        return 0

    def calc_flops(self):
        return 0


class CommOpCost(OpCost):
    """``op_desc``: from ``build_comm_desc``; or ``nbytes`` + ``group_ranks`` given directly."""
    OP_TYPE = "COMM"

    def __init__(self, op=None, op_desc=None, comm_context=None, nbytes=None, group_ranks=None):
        super().__init__(op, op_desc)
        self.comm_context = comm_context or CommContext()
        if op_desc is not None:
            group_ranks = op_desc["group_ranks"]
            nbytes = 0
            for dtype, shape in op_desc["inputs"]["X"]:
                n = _itemsize(dtype)
                for s in shape:
                    n *= s
                nbytes += n
        self.group_ranks, self.comm_count = list(group_ranks or []), int(nbytes or 0)
        self.rank_count = len(self.group_ranks)

    def calc_time(self):
        if self.rank_count <= 1:
            return 0.0
        return self.comm_context.get_alpha(self.group_ranks) + self.volume_factor() * self.comm_count * self.comm_context.get_beta(self.group_ranks)

    def volume_factor(self):
        return 1.0


class CompOpCost(OpCost):
    """``op_desc``: ``{"flops": ..., "bytes": ..., "dtype_bytes": 2 | 4}`` for the local piece of the operator.  The time is
    the roofline of the device: flops over the tensor rate against bytes over the memory rate."""
    OP_TYPE = "COMP"
    FLOP_EFFICIENCY = 1.0
    BYTE_EFFICIENCY = 0.8

    def __init__(self, op=None, op_desc=None, cluster=None):
        super().__init__(op, op_desc)
        self.cluster = cluster

    def _device(self):
        from ..cluster import get_default_cluster
        self.cluster = self.cluster or get_default_cluster()
        return self.cluster.get_all_devices("GPU")[0]

    def calc_flops(self):
        return int(self.op_desc.get("flops", 0))

    def calc_time(self):
        dev = self._device()
        rate = (dev.hp_gflops if self.op_desc.get("dtype_bytes", 4) <= 2 else dev.sp_gflops) * 1e9 * self.FLOP_EFFICIENCY
        t_f = self.op_desc.get("flops", 0) / rate if rate else 0.0
        t_b = self.op_desc.get("bytes", 0) / (dev.hbm_bandwidth * 1e9 * self.BYTE_EFFICIENCY)
        return max(t_f, t_b) + 2e-6            # a launch costs a couple of microseconds

    def calc_memory(self):
        return int(self.op_desc.get("out_bytes", 0))
