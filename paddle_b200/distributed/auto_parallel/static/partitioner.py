"""Per-rank view of a completed program (python/paddle/distributed/auto_parallel/static/partitioner.py and reshard.py):
``Partitioner(dist_context, rank).partition()`` lists, in program order, the communication inserted in front of each
operator (with the ranks of its group) and the operator itself with the shapes of the pieces this rank holds.  The
list is what a rank executes; running it is the job of the distributed-tensor dispatch, which takes the same
decisions from the same rules at run time - the partition is the static record used for inspection, cost and tests."""
from __future__ import annotations

from dataclasses import dataclass

from .completion import local_shape


@dataclass
class DistNode:
    type: str                 # an operator name, or c_allreduce_sum / c_allgather / c_reducescatter / all_to_all / slice
    inputs: list              # (slot, local shape)
    outputs: list
    group_ranks: list = None
    nbytes: int = 0
    is_comm: bool = False

    def __repr__(self):
        if self.is_comm:
            return f"{self.type}(%{self.inputs[0][0]}, ranks={self.group_ranks}, bytes={self.nbytes})"
        return f"{[f'%{s}{sh}' for s, sh in self.outputs]} = {self.type}({[f'%{s}{sh}' for s, sh in self.inputs]})"


_COMM_NAME = {"all_reduce": "c_allreduce_sum", "all_gather": "c_allgather", "reduce_scatter": "c_reducescatter",
              "all_to_all": "all_to_all", "slice": "slice"}


def _coords(rank, mesh_shape):
    out = []
    for s in reversed(mesh_shape):
        out.append(rank % s)
        rank //= s
    return out[::-1]


def group_ranks(rank, axis, mesh_shape):
    """Ranks that share every mesh coordinate of ``rank`` except the one along ``axis`` (row-major numbering)."""
    c = _coords(rank, mesh_shape)
    stride = 1
    for s in mesh_shape[axis + 1:]:
        stride *= s
    base = rank - c[axis] * stride
    return [base + i * stride for i in range(mesh_shape[axis])]


class Resharder:
    """Turns the re-shard records of a ``DistOp`` into communication nodes for one rank."""

    def __init__(self, dist_context, rank_id=0):
        self.ctx, self.rank = dist_context, rank_id

    def reshard_nodes(self, op, outputs=False):
        out = []
        ms = self.ctx.mesh_shape
        for rs in (op.out_reshards if outputs else op.reshards):
            for st in rs.steps:
                out.append(DistNode(_COMM_NAME[st.kind], [(rs.slot, local_shape(rs.src, ms))], [(rs.slot, local_shape(rs.dst, ms))],
                                    group_ranks(self.rank, st.mesh_axis, ms), st.nbytes, True))
        return out


class Partitioner:
    def __init__(self, dist_context, rank_id=0):
        self.ctx, self.rank = dist_context, rank_id
        self._resharder = Resharder(dist_context, rank_id)

    def partition(self, *unused):
        ms = self.ctx.mesh_shape
        nodes = []
        for op in self.ctx.dist_ops:
            nodes.extend(self._resharder.reshard_nodes(op))
            nodes.append(DistNode(op.name, [(s, local_shape(sp, ms)) for s, sp in zip(op.in_slots, op.in_specs)],
                                  [(s, local_shape(sp, ms)) for s, sp in zip(op.out_slots, op.out_specs)]))
            nodes.extend(self._resharder.reshard_nodes(op, outputs=True))
        return nodes

    def local_param_shapes(self):
        return {t: local_shape(self.ctx.tensor_specs[s], self.ctx.mesh_shape) for s, t in self.ctx.params.items()
                if s in self.ctx.tensor_specs}

    def local_slice(self, slot):
        """Index ranges ``[(start, stop), ...]`` of the piece of variable ``slot`` that this rank holds."""
        sp = self.ctx.tensor_specs[slot]
        c = _coords(self.rank, self.ctx.mesh_shape)
        out = []
        for s, m in zip(sp.shape, sp.dims_mapping):
            if m == -1:
                out.append((0, s))
            else:
                step = -(-s // self.ctx.mesh_shape[m])
                out.append((min(s, c[m] * step), min(s, (c[m] + 1) * step)))
        return out

    def to_string(self):
        return "\n".join(repr(n) for n in self.partition())
