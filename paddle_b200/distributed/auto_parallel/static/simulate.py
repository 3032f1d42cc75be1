"""Runs the partition of every rank in ONE process, on whole arrays cut into the pieces the plan gives each rank, with
the collectives done by hand between the pieces - the check that a completed program computes what the serial program
computes (the role of python/paddle/distributed/auto_parallel/static/auto_align_tool.py: find where a parallel run
leaves the serial one).  Covers the operator classes whose local form is the global call on local pieces: matmul,
element-wise, normalisation, softmax, layout changes, sum / mean reductions; others raise ``NotImplementedError``."""
from __future__ import annotations

import torch
from torch.utils import _pytree as pytree

from .partitioner import _coords, group_ranks


class Simulator:
    def __init__(self, dist_context):
        self.ctx = dist_context
        self.ms = dist_context.mesh_shape
        self.n = 1
        for s in self.ms:
            self.n *= s
        self.state = [dict() for _ in range(self.n)]

    # ---------------------------------------------------------------- pieces
    def _cut(self, full, spec, rank):
        c = _coords(rank, self.ms)
        out = full
        for d, m in enumerate(spec.dims_mapping):
            if m != -1:
                step = -(-spec.shape[d] // self.ms[m])
                out = out.narrow(d, c[m] * step, step)
        return out

    def _place(self, slot, full, spec):
        for r in range(self.n):
            self.state[r][slot] = self._cut(full, spec, r).clone()

    def _apply_step(self, slot, st, cur_map, dst):
        a = st.mesh_axis
        done = set()
        for r in range(self.n):
            if r in done:
                continue
            grp = group_ranks(r, a, self.ms)
            done.update(grp)
            parts = [self.state[g][slot] for g in grp]
            if st.kind == "all_reduce":
                tot = sum(parts)
                for g in grp:
                    self.state[g][slot] = tot.clone()
            elif st.kind == "all_gather":
                d = cur_map.index(a)
                tot = torch.cat(parts, d)
                for g in grp:
                    self.state[g][slot] = tot.clone()
            elif st.kind == "reduce_scatter":
                tot = sum(parts)
                d = dst.dims_mapping.index(a)
                for i, g in enumerate(grp):
                    self.state[g][slot] = tot.chunk(len(grp), d)[i].clone()
            elif st.kind == "slice":
                d = dst.dims_mapping.index(a)
                for i, g in enumerate(grp):
                    self.state[g][slot] = self.state[g][slot].chunk(len(grp), d)[i].clone()
            elif st.kind == "all_to_all":
                ds, dd = cur_map.index(a), dst.dims_mapping.index(a)
                tot = torch.cat(parts, ds)
                for i, g in enumerate(grp):
                    self.state[g][slot] = tot.chunk(len(grp), dd)[i].clone()
        if st.kind in ("all_gather",):
            cur_map[cur_map.index(a)] = -1
        elif st.kind in ("reduce_scatter", "slice"):
            cur_map[dst.dims_mapping.index(a)] = a
        elif st.kind == "all_to_all":
            cur_map[cur_map.index(a)] = -1
            cur_map[dst.dims_mapping.index(a)] = a

    # ---------------------------------------------------------------- run
    def run(self, feed, fetch):
        """``feed``: {placeholder name: whole tensor}; ``fetch``: program variables -> whole tensors rebuilt from the pieces
        (partial values summed, split dims concatenated)."""
        from ....static.graph import _Ref
        from .completion import _slot_of
        ctx = self.ctx
        prog = ctx.program
        first_spec = {}
        for op in ctx.dist_ops:
            for rs in op.reshards:
                first_spec.setdefault(rs.slot, rs.src)
            for s, sp in zip(op.in_slots, op.in_specs):
                first_spec.setdefault(s, sp)
        for name, s in ctx.placeholders.items():
            if s in first_spec:
                self._place(s, torch.as_tensor(feed[name]), first_spec[s])
        for s, t in prog._captured.items():
            if s in first_spec:
                self._place(s, t.detach(), first_spec[s])
        for op in ctx.dist_ops:
            if op.kind in ("loss", "embedding", "attention", "other"):
                raise NotImplementedError(f"the simulator has no local form of {op.name}")
            for rs in op.reshards:
                cur = list(rs.src.dims_mapping)
                for st in rs.steps:
                    self._apply_step(rs.slot, st, cur, rs.dst)
            node = op.node
            name = node.name
            for r in range(self.n):
                res = lambda a: self.state[r][a.slot] if isinstance(a, _Ref) else a      # noqa: E731,B023
                args = list(pytree.tree_map(res, node.args))
                kwargs = pytree.tree_map(res, node.kwargs)
                lo = [ctx.local_shape(s, sp) for s, sp in zip(op.out_slots, op.out_specs)]
                if name in ("reshape", "view", "_unsafe_view"):
                    args = [args[0], lo[0]]
                elif name == "mean" and op.out_specs[0].partial_dims:
                    whole = 1
                    for a in op.out_specs[0].partial_dims:
                        whole *= self.ms[a]
                    self.state[r][op.out_slots[0]] = node.func(*args, **kwargs) / whole
                    continue
                with torch.no_grad():
                    out = node.func(*args, **kwargs)
                leaves = [o for o in pytree.tree_leaves(out) if isinstance(o, torch.Tensor)]
                for s, o in zip(op.out_slots, leaves):
                    self.state[r][s] = o
            for rs in op.out_reshards:
                cur = list(rs.src.dims_mapping)
                for st in rs.steps:
                    self._apply_step(rs.slot, st, cur, rs.dst)
        outs = []
        for v in fetch:
            s = _slot_of(prog, v)
            outs.append(self.assemble(s))
        return outs

    def assemble(self, slot):
        sp = self.ctx.tensor_specs[slot]

        def build(axis, fixed):
            if axis == len(self.ms):
                r = 0
                for c, s in zip(fixed, self.ms):
                    r = r * s + c
                return self.state[r][slot]
            pieces = [build(axis + 1, fixed + [i]) for i in range(self.ms[axis])]
            if axis in sp.partial_dims:
                return sum(pieces)
            if axis in sp.dims_mapping:
                return torch.cat(pieces, sp.dims_mapping.index(axis))
            return pieces[0]
        return build(0, [])
