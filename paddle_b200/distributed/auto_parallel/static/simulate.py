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

    def _apply_step(self, vals, st, cur_map, dst):
        """One collective over the per-rank list ``vals`` (in place); ``cur_map`` follows the layout."""
        a = st.mesh_axis
        done = set()
        for r in range(self.n):
            if r in done:
                continue
            grp = group_ranks(r, a, self.ms)
            done.update(grp)
            parts = [vals[g] for g in grp]
            if st.kind == "all_reduce":
                tot = sum(parts)
                new = [tot.clone() for _ in grp]
            elif st.kind == "all_gather":
                tot = torch.cat(parts, cur_map.index(a))
                new = [tot.clone() for _ in grp]
            elif st.kind == "reduce_scatter":
                new = [c.clone() for c in sum(parts).chunk(len(grp), dst.dims_mapping.index(a))]
            elif st.kind == "slice":
                d = dst.dims_mapping.index(a)
                new = [vals[g].chunk(len(grp), d)[i].clone() for i, g in enumerate(grp)]
            elif st.kind == "all_to_all":
                tot = torch.cat(parts, cur_map.index(a))
                new = [c.clone() for c in tot.chunk(len(grp), dst.dims_mapping.index(a))]
            else:
                raise ValueError(st.kind)
            for g, v in zip(grp, new):
                vals[g] = v
        if st.kind == "all_gather":
            cur_map[cur_map.index(a)] = -1
        elif st.kind in ("reduce_scatter", "slice"):
            cur_map[dst.dims_mapping.index(a)] = a
        elif st.kind == "all_to_all":
            cur_map[cur_map.index(a)] = -1
            cur_map[dst.dims_mapping.index(a)] = a

    def _resharded(self, rs):
        vals = [self.state[r][rs.slot] for r in range(self.n)]
        cur = list(rs.src.dims_mapping)
        for st in rs.steps:
            self._apply_step(vals, st, cur, rs.dst)
        return vals

    # ---------------------------------------------------------------- run
    def run(self, feed, fetch):
        """``feed``: {placeholder name: whole tensor}; ``fetch``: program variables -> whole tensors rebuilt from the pieces
        (partial values summed, split dims concatenated)."""
        from ....static.graph import _Ref
        from .completion import _slot_of
        ctx = self.ctx
        prog = ctx.program
        first_spec = {s: sp for s, sp in ctx.tensor_specs.items() if not sp.partial_dims}
        for name, s in ctx.placeholders.items():
            if s in first_spec:
                self._place(s, torch.as_tensor(feed[name]), first_spec[s])
        for s, t in prog._captured.items():
            if s in first_spec:
                self._place(s, t.detach(), first_spec[s])
        for op in ctx.dist_ops:
            if op.kind == "other" and any(m != -1 for sp in op.in_specs for m in sp.dims_mapping):
                raise NotImplementedError(f"the simulator has no local form of {op.name}")
            local = {rs.slot: self._resharded(rs) for rs in op.reshards}      # what THIS operator sees; the variable stays
            node = op.node
            name = node.name
            for r in range(self.n):
                res = lambda a: (local[a.slot][r] if a.slot in local else self.state[r][a.slot]) if isinstance(a, _Ref) else a   # noqa: E731,B023,E501
                args = list(pytree.tree_map(res, node.args))
                kwargs = pytree.tree_map(res, node.kwargs)
                lo = [ctx.local_shape(s, sp) for s, sp in zip(op.out_slots, op.out_specs)]
                if op.kind == "embedding" and op.in_specs[1].dims_mapping[0] != -1:
                    # rows of the table are split: look up what this rank owns, zeros elsewhere (the output is partial)
                    a = op.in_specs[1].dims_mapping[0]
                    rows = args[1].shape[0]
                    ids = args[0] - _coords(r, self.ms)[a] * rows
                    own = (ids >= 0) & (ids < rows)
                    with torch.no_grad():
                        out = node.func(ids.clamp(0, rows - 1), *args[1:], **kwargs) * own.unsqueeze(-1)
                    self.state[r][op.out_slots[0]] = out
                    continue
                if op.kind == "loss" and any(m != -1 and sh > 1 and i == (1 if op.in_specs[0].ndim > 1 else 0)
                                             for i, (m, sh) in enumerate(zip(op.in_specs[0].dims_mapping, op.in_specs[0].shape))):
                    # the class dim is split: the operator reduces over that mesh axis inside; here the pieces of the
                    # group are put together and every rank of the group computes the same loss
                    cd = 1 if op.in_specs[0].ndim > 1 else 0
                    a = op.in_specs[0].dims_mapping[cd]
                    slot = op.in_slots[0]
                    src = local[slot] if slot in local else [self.state[g][slot] for g in range(self.n)]
                    args[0] = torch.cat([src[g] for g in group_ranks(r, a, self.ms)], cd)
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
                for r, v in enumerate(self._resharded(rs)):
                    self.state[r][rs.slot] = v
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
