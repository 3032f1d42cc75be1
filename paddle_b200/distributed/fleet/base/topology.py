"""Hybrid-parallel topology (python/paddle/distributed/fleet/base/topology.py:70 ``CommunicateTopology``,
:189 ``HybridCommunicateGroup``).  Five axes named data / pipe / sharding / sep / model in a configurable
order; rank <-> coordinate is a cartesian product; one communication group per axis value plus the
fused dp x sep and pp x mp groups and the pipeline neighbours."""
from __future__ import annotations

import collections
import itertools
from functools import reduce

from ... import collective as C


class ParallelMode:
    DATA_PARALLEL = 0
    TENSOR_PARALLEL = 1
    PIPELINE_PARALLEL = 2
    SHARDING_PARALLEL = 3
    SEGMENT_PARALLEL = 4


class CommunicateTopology:
    def __init__(self, hybrid_group_names=("data", "pipe", "sharding", "sep", "model"), dims=(1, 1, 1, 1, 1)):
        self._parallel_names = list(hybrid_group_names)
        self._dims = list(dims)
        self.coordinate = collections.namedtuple("Coordinate", self._parallel_names)
        self._world_size = reduce(lambda a, b: a * b, self._dims, 1)
        ranges = [range(d) for d in self._dims]
        all_coord = [self.coordinate(*c) for c in itertools.product(*ranges)]
        self._coord2rank = dict(zip(all_coord, range(len(all_coord))))
        self._rank2coord = dict(zip(self._coord2rank.values(), self._coord2rank.keys()))

    def get_hybrid_group_names(self):
        return self._parallel_names

    def get_dim(self, axis_name):
        return self._dims[self._parallel_names.index(axis_name)]

    get_dim_size = get_dim

    def world_size(self):
        return self._world_size

    def get_rank(self, **args):
        return self._coord2rank[self.coordinate(**args)]

    def get_coord(self, rank):
        return self._rank2coord[rank]

    def get_axis_list(self, axis_name, index):
        axis = self._parallel_names.index(axis_name)
        return sorted(r for c, r in self._coord2rank.items() if c[axis] == index)

    def get_comm_list(self, axis_name):
        """All groups along ``axis_name``: ranks that differ only in that coordinate."""
        axis = self._parallel_names.index(axis_name)
        others = [range(d) for i, d in enumerate(self._dims) if i != axis]
        out = []
        for fixed in itertools.product(*others):
            ranks = []
            for v in range(self._dims[axis]):
                coord = list(fixed)
                coord.insert(axis, v)
                ranks.append(self._coord2rank[self.coordinate(*coord)])
            out.append(ranks)
        return out

    def get_fused_ranks(self, fused_axis):
        axes = [self._parallel_names.index(a) for a in fused_axis]
        others = [i for i in range(len(self._dims)) if i not in axes]
        out = []
        for fixed in itertools.product(*[range(self._dims[i]) for i in others]):
            ranks = []
            for vals in itertools.product(*[range(self._dims[i]) for i in axes]):
                coord = [0] * len(self._dims)
                for i, v in zip(others, fixed):
                    coord[i] = v
                for i, v in zip(axes, vals):
                    coord[i] = v
                ranks.append(self._coord2rank[self.coordinate(*coord)])
            out.append(sorted(ranks))
        return out

    def get_rank_from_stage(self, global_rank, **kwargs):
        coord = self.get_coord(global_rank)._replace(**kwargs)
        return self._coord2rank[coord]


class HybridCommunicateGroup:
    def __init__(self, topology: CommunicateTopology):
        self._topo = topology
        self.nranks = C.get_world_size()
        self.global_rank = C.get_rank()
        names = topology.get_hybrid_group_names()
        self._dp_degree = topology.get_dim("data")
        self._mp_degree = topology.get_dim("model")
        self._pp_degree = topology.get_dim("pipe")
        self._sharding_degree = topology.get_dim("sharding")
        self._sep_degree = topology.get_dim("sep") if "sep" in names else 1
        assert topology.world_size() == self.nranks, (
            f"hybrid degrees multiply to {topology.world_size()} but the job has {self.nranks} ranks")
        coord = topology.get_coord(self.global_rank)
        self._data_parallel_id = coord.data
        self._model_parallel_id = coord.model
        self._sharding_parallel_id = coord.sharding
        self._sep_parallel_id = coord.sep if "sep" in names else 0
        self.stage_id = coord.pipe
        self._dp_group, self._dp_comm_group = self._set_comm_group("data")
        self._mp_group, self._mp_comm_group = self._set_comm_group("model")
        self._pp_group, self._pp_comm_group = self._set_comm_group("pipe")
        self._sharding_group, self._sharding_comm_group = self._set_comm_group("sharding")
        self._sep_group, self._sep_comm_group = (self._set_comm_group("sep") if "sep" in names and self._sep_degree > 1
                                                 else ([self.global_rank], None))
        self._check_group, self._check_comm_group = self._set_check_group("data")
        if self._sep_degree > 1:
            self._dp_sep_group, self._dp_sep_comm_group = self._set_fused_group(["data", "sep"])
        else:
            self._dp_sep_group, self._dp_sep_comm_group = self._dp_group, self._dp_comm_group
        if self._pp_degree > 1 and self._mp_degree > 1:
            self._pp_mp_group, self._pp_mp_comm_group = self._set_fused_group(["pipe", "model"])
        else:
            self._pp_mp_group = self._pp_mp_comm_group = None
        # pipeline neighbours
        self.is_first_stage = self.stage_id == 0
        self.is_last_stage = self.stage_id == self._pp_degree - 1
        if self._pp_degree > 1:
            self.next_rank = topology.get_rank_from_stage(self.global_rank, pipe=(self.stage_id + 1) % self._pp_degree)
            self.prev_rank = topology.get_rank_from_stage(self.global_rank, pipe=(self.stage_id - 1) % self._pp_degree)
            C.all_reduce(_warmup_tensor(), group=self._pp_comm_group)   # create the communicator early
        else:
            self.next_rank = self.prev_rank = self.global_rank

    def _set_comm_group(self, axis):
        mine, mine_g = None, None
        degree = self._topo.get_dim(axis)
        for ranks in self._topo.get_comm_list(axis):
            g = C.new_group(ranks) if degree > 1 else None
            if self.global_rank in ranks:
                mine = ranks
                mine_g = g if g is not None else C.Group(0, -1, ranks, None)
        return mine, mine_g

    def _set_check_group(self, axis):
        # ranks sharing the same data-parallel index: used to agree on found_inf
        ranks = self._topo.get_axis_list(axis, self._data_parallel_id)
        if len(ranks) == self.nranks:
            return ranks, C._get_default_group()
        mine = None
        for idx in range(self._topo.get_dim(axis)):
            rs = self._topo.get_axis_list(axis, idx)
            g = C.new_group(rs)
            if self.global_rank in rs:
                mine = g
        return ranks, mine

    def _set_fused_group(self, axes):
        mine, mine_g = None, None
        for ranks in self._topo.get_fused_ranks(axes):
            g = C.new_group(ranks)
            if self.global_rank in ranks:
                mine, mine_g = ranks, g
        return mine, mine_g

    def get_parallel_mode(self):
        if self._pp_degree > 1:
            return ParallelMode.PIPELINE_PARALLEL
        if self._mp_degree > 1:
            return ParallelMode.TENSOR_PARALLEL
        if self._sep_degree > 1:
            return ParallelMode.SEGMENT_PARALLEL
        if self._sharding_degree > 1:
            return ParallelMode.SHARDING_PARALLEL
        return ParallelMode.DATA_PARALLEL

    def topology(self):
        return self._topo

    def get_global_rank(self):
        return self.global_rank

    # data parallel
    def get_data_parallel_rank(self): return self._data_parallel_id
    def get_data_parallel_world_size(self): return self._dp_degree
    def get_data_parallel_group(self): return self._dp_comm_group
    def get_data_parallel_group_src_rank(self): return self._dp_group[0]
    # model parallel
    def get_model_parallel_rank(self): return self._model_parallel_id
    def get_model_parallel_world_size(self): return self._mp_degree
    def get_model_parallel_group(self): return self._mp_comm_group
    def get_model_parallel_group_src_rank(self): return self._mp_group[0]
    # pipeline
    def get_stage_id(self): return self.stage_id
    def get_pipe_parallel_rank(self): return self.stage_id
    def get_pipe_parallel_world_size(self): return self._pp_degree
    def get_pipe_parallel_group(self): return self._pp_comm_group
    def get_p2p_groups(self): return None
    # sharding
    def get_sharding_parallel_rank(self): return self._sharding_parallel_id
    def get_sharding_parallel_world_size(self): return self._sharding_degree
    def get_sharding_parallel_group(self): return self._sharding_comm_group
    def get_sharding_parallel_group_src_rank(self): return self._sharding_group[0]
    # sep
    def get_sep_parallel_rank(self): return self._sep_parallel_id
    def get_sep_parallel_world_size(self): return self._sep_degree
    def get_sep_parallel_group(self): return self._sep_comm_group
    def get_dp_sep_parallel_group(self): return self._dp_sep_comm_group
    def get_pp_mp_parallel_group(self): return self._pp_mp_comm_group
    def get_check_parallel_group(self, sharding=False): return self._check_comm_group

    def get_rank_from_stage(self, stage_id, **kwargs):
        return self._topo.get_rank_from_stage(self.global_rank, pipe=stage_id, **kwargs)


def _warmup_tensor():
    import torch
    from ...._core import dtype as _dt
    return torch.zeros(1, device=_dt.default_device())
