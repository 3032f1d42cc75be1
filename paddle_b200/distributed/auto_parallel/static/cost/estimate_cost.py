"""Cost of a completed program (python/paddle/distributed/auto_parallel/static/cost/estimate_cost.py): walks the
``DistOp`` list of a ``DistContext``, prices the local piece of every operator and every re-shard in front of it with
the operator cost classes, mirrors the communication for the backward pass, adds the gradient synchronisation of the
parameters and sums parameter, gradient, optimizer-state and activation bytes into the peak memory of one rank."""
from __future__ import annotations

from .base_cost import CommContext, Cost, _g_op_cost_factory
from . import comm_op_cost, comp_op_cost  # noqa: F401  (register the classes)

_BWD_FACTOR = {"matmul": 2.0, "attention": 2.5, "embedding": 1.0, "norm": 1.5, "softmax": 1.0, "loss": 1.0, "reduce": 1.0,
               "elementwise": 1.0, "layout": 0.0, "other": 1.0}
_MIRROR = {"all_gather": "reduce_scatter", "reduce_scatter": "all_gather", "all_reduce": None, "all_to_all": "all_to_all",
           "slice": "all_gather"}


def _prod(xs):
    n = 1
    for x in xs:
        n *= x
    return n


class CostEstimator:
    _special_op_type = ["fused_attention", "fused_feedforward"]

    def __init__(self, dist_context, cluster=None, mode="train", grad_sync_overlap=0.7, loop_count=None):
        from ..cluster import get_default_cluster
        self.ctx = dist_context
        self.cluster = cluster or get_default_cluster(device_count=max(1, _prod(dist_context.mesh_shape)))
        self.mode = mode
        self.grad_sync_overlap = grad_sync_overlap
        self.comm_context = CommContext(self.cluster)
        self.detailed = []
        self._global_cost = None
        self.max_memory = 0
        self.parts = {}

    # ---------------------------------------------------------------- helpers
    def _group(self, axis):
        ms = self.ctx.mesh_shape
        stride = _prod(ms[axis + 1:])
        return [i * stride for i in range(ms[axis])]

    def _comm_time(self, kind, axis, nbytes):
        if kind in (None, "slice") or self.ctx.mesh_shape[axis] <= 1:
            return 0.0
        return _g_op_cost_factory[kind](comm_context=self.comm_context, nbytes=nbytes, group_ranks=self._group(axis)).time

    def _op_desc(self, op):
        c = self.ctx
        in_b = sum(c.nbytes(s, sp) for s, sp in zip(op.in_slots, op.in_specs))
        out_b = sum(c.nbytes(s, sp) for s, sp in zip(op.out_slots, op.out_specs))
        item = min([c.dtypes[s].itemsize for s in op.in_slots if c.dtypes[s].is_floating_point] or [4])
        flops = 0
        if op.kind == "matmul" and op.out_specs:
            xi = op.attrs.get("x", 0)
            k_full = op.attrs["k"]
            x = op.in_specs[xi]
            m = x.dims_mapping[-1]
            k_local = k_full if (m == -1 or op.name.startswith("conv")) else -(-k_full // c.mesh_shape[m])
            flops = 2 * _prod(c.local_shape(op.out_slots[0], op.out_specs[0])) * k_local
        elif op.kind == "attention":
            b, h, s, d = c.local_shape(op.in_slots[0], op.in_specs[0])
            t = c.local_shape(op.in_slots[1], op.in_specs[1])[2]
            flops = int(4 * b * h * s * t * d * (0.5 if op.attrs.get("causal") else 1.0))
        elif op.kind != "layout":
            flops = out_b // max(item, 1)
        return {"flops": flops, "bytes": in_b + out_b, "out_bytes": out_b, "dtype_bytes": item}

    # ---------------------------------------------------------------- the estimate
    def estimate_cost(self):
        c = self.ctx
        train = self.mode == "train"
        comp = comm = sync = 0.0
        flops = 0
        act_bytes = peak_act = 0
        self.detailed = []
        for op in c.dist_ops:
            desc = self._op_desc(op)
            cls = _g_op_cost_factory.get(op.kind, _g_op_cost_factory["other"])
            oc = cls(op=op, op_desc=desc, cluster=self.cluster)
            t_f = oc.time
            t_b = t_f * _BWD_FACTOR.get(op.kind, 1.0) if train else 0.0
            t_c = 0.0
            for rs in op.reshards + op.out_reshards:
                no_grad = rs.slot in c.placeholders.values() or rs.slot in c.params
                for st in rs.steps:
                    t_c += self._comm_time(st.kind, st.mesh_axis, st.nbytes)
                    if train and not no_grad:
                        nb = st.nbytes if st.kind != "slice" else c.nbytes(rs.slot, rs.src)
                        t_c += self._comm_time(_MIRROR[st.kind], st.mesh_axis, nb)
            if train:
                for st in op.backward_comm:
                    t_c += self._comm_time(st.kind, st.mesh_axis, st.nbytes)
            t_s = 0.0
            if train:
                for s, axes in op.grad_sync.items():
                    for a in axes:
                        t_s += self._comm_time("all_reduce", a, c.nbytes(s, op.in_specs[op.in_slots.index(s)]))
            comp += t_f + t_b
            comm += t_c
            sync += t_s
            flops += desc["flops"] * (1 + (_BWD_FACTOR.get(op.kind, 1.0) if train else 0))
            if op.kind != "layout":
                act_bytes += desc["out_bytes"]
                peak_act = max(peak_act, desc["bytes"])
            self.detailed.append({"op": op.name, "kind": op.kind, "compute": t_f + t_b, "comm": t_c, "grad_sync": t_s,
                                  "flops": desc["flops"], "reshards": [(st.kind, st.mesh_axis, st.nbytes) for rs in op.reshards + op.out_reshards for st in rs.steps]})
        p_bytes = o_bytes = 0
        for s, t in c.params.items():
            sp = c.tensor_specs.get(s)
            if sp is None:
                continue
            n = c.nbytes(s, sp)
            p_bytes += n
            if train:
                elems = n // t.dtype.itemsize
                o_bytes += n + elems * (12 if t.dtype.itemsize < 4 else 8)          # gradient + two moments (+ fp32 master)
        memory = p_bytes + o_bytes + (act_bytes if train else peak_act)
        self.max_memory = memory
        exposed_sync = sync * (1.0 - self.grad_sync_overlap)
        self.parts = {"compute": comp, "comm": comm, "grad_sync": sync, "grad_sync_exposed": exposed_sync,
                      "param_bytes": p_bytes, "optimizer_bytes": o_bytes, "activation_bytes": act_bytes if train else peak_act}
        self._global_cost = Cost(comp + comm + exposed_sync, memory, flops)
        return self._global_cost

    global_cost = property(lambda self: self._global_cost or self.estimate_cost())

    def get_op_cost(self):
        return self.detailed

    def pretty_print_cost(self):
        if self._global_cost is None:
            self.estimate_cost()
        rows = [f"{'op':<28}{'kind':<12}{'compute(us)':>12}{'comm(us)':>10}{'sync(us)':>10}  reshards"]
        for d in self.detailed:
            if d["compute"] or d["comm"] or d["grad_sync"]:
                rows.append(f"{d['op']:<28}{d['kind']:<12}{d['compute'] * 1e6:>12.1f}{d['comm'] * 1e6:>10.1f}{d['grad_sync'] * 1e6:>10.1f}  "
                            + ", ".join(f"{k}@{a}" for k, a, _ in d["reshards"]))
        rows.append(f"total: {self._global_cost}  parts: " + ", ".join(f"{k}={v:.3e}" for k, v in self.parts.items()))
        text = "\n".join(rows)
        print(text)
        return text


def get_cost_from_engine(engine, mode="train"):
    """(time in seconds, memory in bytes) of the plan an ``Engine`` holds; ``None`` before it planned one."""
    plan = getattr(engine, "_plan", None)
    if plan is None:
        return None
    return plan.cost.time, plan.cost.memory
