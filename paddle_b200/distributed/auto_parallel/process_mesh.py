"""``ProcessMesh`` and placements (python/paddle/distributed/auto_parallel/process_mesh.py:80,
placement_type.py; C++ side paddle/phi/core/distributed/auto_parallel/process_mesh.h, placement_types.h)."""
from __future__ import annotations

import numpy as np

from .. import collective as C


class ReduceType:
    kRedSum, kRedMax, kRedMin, kRedProd, kRedAvg, kRedAny, kRedAll = range(7)


class Placement:
    def is_shard(self, dim=None):
        return False

    def is_replicated(self):
        return False

    def is_partial(self):
        return False


class Shard(Placement):
    def __init__(self, dim):
        self.dim = int(dim)

    def get_dim(self):
        return self.dim

    def is_shard(self, dim=None):
        return dim is None or dim == self.dim

    def __eq__(self, o):
        return isinstance(o, Shard) and o.dim == self.dim

    def __hash__(self):
        return hash(("S", self.dim))

    def __repr__(self):
        return f"Shard(dim={self.dim})"


class Replicate(Placement):
    def is_replicated(self):
        return True

    def __eq__(self, o):
        return isinstance(o, Replicate)

    def __hash__(self):
        return hash("R")

    def __repr__(self):
        return "Replicate()"


class Partial(Placement):
    def __init__(self, reduce_type=ReduceType.kRedSum):
        self.reduce_type = reduce_type

    def is_partial(self):
        return True

    def __eq__(self, o):
        return isinstance(o, Partial) and o.reduce_type == self.reduce_type

    def __hash__(self):
        return hash(("P", self.reduce_type))

    def __repr__(self):
        return f"Partial(reduce_type={self.reduce_type})"


_AXIS_GROUPS = {}
_global_mesh = None


class ProcessMesh:
    def __init__(self, mesh=None, dim_names=None, shape=None, process_ids=None):
        if mesh is None:
            mesh = np.asarray(process_ids).reshape(shape)
        self._mesh = np.asarray(mesh, dtype=np.int64)
        if self._mesh.ndim == 0:
            self._mesh = self._mesh.reshape(1)
        self._dim_names = list(dim_names) if dim_names is not None else [f"d{i}" for i in range(self._mesh.ndim)]
        assert len(self._dim_names) == self._mesh.ndim and len(set(self._dim_names)) == self._mesh.ndim
        assert len(set(self._mesh.flatten().tolist())) == self._mesh.size, "process ids must be unique"

    mesh = property(lambda self: self._mesh.tolist())
    shape = property(lambda self: list(self._mesh.shape))
    ndim = property(lambda self: self._mesh.ndim)
    dim_names = property(lambda self: list(self._dim_names))
    process_ids = property(lambda self: self._mesh.flatten().tolist())

    def get_dim_size(self, dim):
        return self._mesh.shape[self._axis(dim)]

    def _axis(self, dim):
        return self._dim_names.index(dim) if isinstance(dim, str) else int(dim)

    def __contains__(self, rank):
        return int(rank) in self.process_ids

    def coord_of(self, rank):
        idx = np.argwhere(self._mesh == rank)
        return None if len(idx) == 0 else tuple(int(i) for i in idx[0])

    def get_mesh_with_dim(self, dim_name, index=None):
        a = self._axis(dim_name)
        order = [a] + [i for i in range(self.ndim) if i != a]
        m = self._mesh.transpose(order)
        names = [self._dim_names[i] for i in order]
        if index is not None:
            return ProcessMesh(m[index], names[1:])
        return ProcessMesh(m, names)

    def get_submesh_with_dim(self, dim_name):
        """The 1-D mesh along ``dim_name`` that contains the calling rank."""
        a = self._axis(dim_name)
        c = self.coord_of(C.get_rank())
        sl = tuple(slice(None) if i == a else c[i] for i in range(self.ndim))
        return ProcessMesh(self._mesh[sl], [self._dim_names[a]])

    def __getitem__(self, idx):
        sub = self._mesh[idx]
        idx_t = idx if isinstance(idx, tuple) else (idx,)
        kept = [n for i, n in enumerate(self._dim_names) if i >= len(idx_t) or isinstance(idx_t[i], slice)]
        if sub.ndim == 0:
            return ProcessMesh(sub.reshape(1), ["d0"])
        return ProcessMesh(sub, kept)

    def __eq__(self, o):
        return isinstance(o, ProcessMesh) and self._mesh.shape == o._mesh.shape and \
            (self._mesh == o._mesh).all() and self._dim_names == o._dim_names

    def __hash__(self):
        return hash((self._mesh.tobytes(), tuple(self._mesh.shape), tuple(self._dim_names)))

    def __repr__(self):
        return f"ProcessMesh(mesh={self.mesh}, dim_names={self._dim_names})"

    # ------------------------------------------------------------------ communication groups
    def get_group(self, dim=None):
        """Process group of the calling rank along one mesh axis.  Every rank creates the groups of ALL lines
        along that axis in the same order (group creation is collective); results are cached."""
        a = 0 if dim is None else self._axis(dim)
        key = (self._mesh.tobytes(), tuple(self._mesh.shape), a)
        if key not in _AXIS_GROUPS:
            moved = np.moveaxis(self._mesh, a, -1).reshape(-1, self._mesh.shape[a])
            mine = None
            me = C.get_rank()
            for line in moved:
                ranks = [int(r) for r in line]
                if len(ranks) == C.get_world_size() and sorted(ranks) == list(range(len(ranks))) and ranks == sorted(ranks):
                    g = C._get_default_group()
                else:
                    g = C.new_group(ranks)
                if me in ranks:
                    mine = g
            _AXIS_GROUPS[key] = mine
        return _AXIS_GROUPS[key]

    def axis_rank(self, axis):
        c = self.coord_of(C.get_rank())
        return None if c is None else c[axis]


def set_mesh(mesh):
    global _global_mesh
    _global_mesh = mesh


def get_mesh():
    return _global_mesh
