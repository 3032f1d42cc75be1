"""Completion of a partially annotated program (python/paddle/distributed/auto_parallel/static/completion.py).

The user (or the planner) fixes the sharding of a few variables of a recorded program - the batch dim of the data, the
weights of some layers - and ``Completer.complete_forward_annotation`` derives the sharding of every other variable
and, per operator, the layout its inputs must be brought into: each operator is mapped to a rule of the SPMD rule
registry (``spmd_rules.py``), the rule merges the inputs' annotations into a consistent set, and every difference
between what an input has and what the operator needs becomes a re-shard step (all-gather, all-reduce,
reduce-scatter, all-to-all, or a local slice).  Operators without a rule take whole inputs.

The result is a ``DistContext``: ``tensor_specs[slot]`` (``DistTensorSpec`` per variable) and ``dist_ops`` (one
``DistOp`` per operator with the input / output specs, the re-shards in front of it, its class for the cost model, and
the mesh axes over which the gradients of its parameters must be summed)."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch.utils import _pytree as pytree

from ..spmd_rules import DistTensorSpec, get_phi_spmd_rule


@dataclass
class CommStep:
    kind: str            # all_gather | all_reduce | reduce_scatter | all_to_all | slice
    mesh_axis: int
    nbytes: int          # bytes of the local buffer that takes part (the gathered one for all_gather)


@dataclass
class Reshard:
    slot: int
    src: DistTensorSpec
    dst: DistTensorSpec
    steps: list


@dataclass
class DistOp:
    node: object
    name: str
    kind: str                                  # matmul | attention | embedding | norm | softmax | loss | reduce | elementwise | layout | other
    in_slots: list
    in_specs: list                             # what the operator consumes (after the re-shards)
    out_slots: list
    out_specs: list
    reshards: list = field(default_factory=list)           # in front of the operator, on its inputs
    out_reshards: list = field(default_factory=list)       # behind it, where an output was pinned to another layout
    param_slots: list = field(default_factory=list)
    grad_sync: dict = field(default_factory=dict)      # param slot -> mesh axes over which its gradient is summed
    backward_comm: list = field(default_factory=list)  # CommStep: collectives only the backward pass needs
    attrs: dict = field(default_factory=dict)


class DistContext:
    def __init__(self, program, mesh_shape, dim_names=None):
        self.program, self.mesh_shape = program, list(mesh_shape)
        self.dim_names = list(dim_names) if dim_names else [f"d{i}" for i in range(len(mesh_shape))]
        self.tensor_specs = {}
        self.dist_ops = []
        self.shapes, self.dtypes, self.params, self.placeholders = {}, {}, {}, {}

    def get_tensor_dist_attr(self, var):
        return self.tensor_specs.get(_slot_of(self.program, var))

    def local_shape(self, slot, spec=None):
        spec = spec or self.tensor_specs[slot]
        return local_shape(spec, self.mesh_shape)

    def nbytes(self, slot, spec=None):
        n = 1
        for s in self.local_shape(slot, spec):
            n *= s
        return n * self.dtypes.get(slot, torch.float32).itemsize


def local_shape(spec, mesh_shape):
    return [s if m == -1 else -(-s // mesh_shape[m]) for s, m in zip(spec.shape, spec.dims_mapping)]


def _slot_of(program, var):
    if isinstance(var, int):
        return var
    if isinstance(var, str):
        if var in program._placeholders:
            return program._placeholders[var][0]
        t = program._names.get(var)
        if t is None:
            raise KeyError(f"no variable named {var!r} in the program")
        var = t
    s = program._slot_of_id.get(id(var))
    if s is None:
        from ....static.graph import _key
        s = program._slot_of_key.get(_key(var))
    if s is None:
        raise KeyError("the tensor is not a variable of the program")
    return s


# ------------------------------------------------------------------------------------------------ operator classes
_ELEMENTWISE = {
    "add", "sub", "mul", "div", "true_divide", "rsub", "pow", "maximum", "minimum", "fmax", "fmin", "gelu", "relu", "relu6", "silu", "tanh",
    "sigmoid", "exp", "expm1", "log", "log1p", "log2", "sqrt", "rsqrt", "neg", "abs", "dropout", "float", "long", "int", "half",
    "bfloat16", "double", "bool", "to", "type_as", "clamp", "clip", "clamp_min", "clamp_max", "ne", "eq", "gt", "lt", "ge", "le", "where",
    "masked_fill", "sin", "cos", "erf", "square", "reciprocal", "contiguous", "clone", "detach", "leaky_relu", "elu", "softplus",
    "hardswish", "hardsigmoid", "hardtanh", "mish", "logsigmoid", "sign", "floor", "ceil", "round", "logical_and", "logical_or", "logical_not",
    "logical_xor", "bitwise_and", "bitwise_or", "bitwise_not", "bitwise_xor", "lerp", "addcmul", "addcdiv", "nan_to_num", "isfinite",
    "isnan", "isinf", "fill", "zero", "copy", "alias", "floor_divide", "remainder", "fmod", "atan2", "selu", "celu", "threshold", "tan",
    "sinh", "cosh", "asin", "acos", "atan", "trunc", "frac", "positive", "zeros_like", "ones_like", "full_like", "rand_like", "randn_like",
    "empty_like", "requires_grad", "lgamma", "digamma", "erfinv", "sigmoid_", "mse_loss_none", "glu_pair",
}
_REDUCE = {"sum", "mean", "amax", "amin", "max", "min", "prod", "all", "any", "logsumexp", "norm", "var", "std"}
_LAYOUT_RESHAPE = {"reshape", "view", "_unsafe_view", "flatten", "unflatten", "view_as", "reshape_as"}
_ATTR_PERM = {"mT": "last2", "T": "reverse", "mH": "last2", "H": "reverse"}


def _refs(obj):
    from ....static.graph import _Ref
    return [a for a in pytree.tree_leaves(obj) if isinstance(a, _Ref)]


def _is_ref(a):
    from ....static.graph import _Ref
    return isinstance(a, _Ref)


def _arg(node, pos, name, default=None):
    if name in node.kwargs:
        return node.kwargs[name]
    return node.args[pos] if len(node.args) > pos else default


def _flat(nodes):
    """Recompute / mixed-precision segments made by the program passes are planned node by node."""
    for n in nodes:
        if getattr(n, "mode", None) in ("recompute", "autocast") and hasattr(n, "nodes"):
            yield from _flat(n.nodes)
        else:
            yield n


class Completer:
    def __init__(self, program, mesh_shape, dim_names=None, assume_dtype=None):
        """``assume_dtype``: price floating-point variables as this dtype (a program recorded in float32 that will run
        under automatic mixed precision in bfloat16)."""
        self.ctx = DistContext(program, mesh_shape, dim_names)
        self.program = program
        self._assume_dtype = assume_dtype
        self._annotated = {}
        self.pre_op_hook = None              # called as hook(completer, node) before an operator is inferred
        self.prefer_scatter = {}             # mesh axis -> tensor dim: a partial sum entering an element-wise operator is
        #                                      reduce-scattered along that dim instead of all-reduced (sequence parallel)
        self._cur_elementwise = False
        self._collect_vars()

    dist_context = property(lambda self: self.ctx)

    # ---------------------------------------------------------------- variables
    def _collect_vars(self):
        p, c = self.program, self.ctx
        for t in p._keep:
            s = p._slot_of_id.get(id(t))
            if s is not None:
                c.shapes[s], c.dtypes[s] = list(t.shape), t.dtype
        for s, t in p._captured.items():
            c.shapes[s], c.dtypes[s] = list(t.shape), t.dtype
            if isinstance(t, torch.nn.Parameter) or getattr(t, "trainable", False) or t.requires_grad:
                c.params[s] = t
        for name, (s, t) in p._placeholders.items():
            c.placeholders[name] = s
            c.shapes[s], c.dtypes[s] = list(t.shape), t.dtype
        if self._assume_dtype is not None:
            for s, d in c.dtypes.items():
                if d.is_floating_point:
                    c.dtypes[s] = self._assume_dtype

    def annotate(self, var, dims_mapping):
        """Fix the sharding of a variable (a program variable, its name, or its slot number)."""
        s = _slot_of(self.program, var)
        if len(dims_mapping) != len(self.ctx.shapes[s]):
            raise ValueError(f"dims_mapping {dims_mapping} does not fit a variable of shape {self.ctx.shapes[s]}")
        for d, m in enumerate(dims_mapping):
            if m != -1 and self.ctx.shapes[s][d] % self.ctx.mesh_shape[m] != 0:
                raise ValueError(f"dim {d} of size {self.ctx.shapes[s][d]} cannot be split over mesh axis {m} "
                                 f"of size {self.ctx.mesh_shape[m]}")
        self._annotated[s] = list(dims_mapping)
        return self

    def _spec(self, slot):
        sp = self.ctx.tensor_specs.get(slot)
        if sp is None:
            sp = DistTensorSpec(self.ctx.shapes[slot], self._annotated.get(slot, [-1] * len(self.ctx.shapes[slot])))
            self.ctx.tensor_specs[slot] = sp
        return sp

    # ---------------------------------------------------------------- re-shard between two specs
    def _reshard(self, slot, src, dst):
        steps = []
        ms = self.ctx.mesh_shape
        cur = list(src.dims_mapping)
        item = self.ctx.dtypes.get(slot, torch.float32).itemsize

        def nbytes(mapping):
            n = item
            for s, m in zip(src.shape, mapping):
                n *= s if m == -1 else -(-s // ms[m])
            return n
        axes = [a for a in range(len(ms)) if ms[a] > 1]
        want = lambda a: dst.dims_mapping.index(a) if a in dst.dims_mapping else None      # noqa: E731
        for a in axes:                                   # partial sums first
            if a in src.partial_dims:
                d_dim = want(a)
                if d_dim is not None and cur[d_dim] == -1:
                    steps.append(CommStep("reduce_scatter", a, nbytes(cur)))
                    cur[d_dim] = a
                else:
                    steps.append(CommStep("all_reduce", a, nbytes(cur)))
        for a in axes:                                   # splits that sit on the wrong dim: move or gather them
            if a not in cur:
                continue
            s_dim, d_dim = cur.index(a), want(a)
            if s_dim == d_dim:
                continue
            if d_dim is not None and cur[d_dim] == -1:
                steps.append(CommStep("all_to_all", a, nbytes(cur)))
                cur[s_dim], cur[d_dim] = -1, a
            else:
                cur[s_dim] = -1
                steps.append(CommStep("all_gather", a, nbytes(cur)))
        for a in axes:                                   # what is still missing is a local slice
            d_dim = want(a)
            if d_dim is not None and a not in cur:
                cur[d_dim] = a
                steps.append(CommStep("slice", a, 0))
        return Reshard(slot, src, dst, steps) if steps else None

    # ---------------------------------------------------------------- one operator
    def _infer(self, node):
        """-> (kind, rule result (new_in, outs) over the tensor inputs in ``slots`` order, slots, attrs)."""
        name = node.name.rstrip("_") if not node.name.startswith("__") else node.name
        refs = _refs((node.args, node.kwargs))
        slots = [r.slot for r in refs]
        self._cur_elementwise = name in _ELEMENTWISE
        specs = [self._strip(self._spec(s)) for s in slots]
        out_shapes = [self.ctx.shapes[s] for s in node.out_slots]
        R = get_phi_spmd_rule
        if not slots:
            return "other", ([], [DistTensorSpec(sh, [-1] * len(sh)) for sh in out_shapes]), slots, {}
        if name in ("matmul", "mm", "bmm", "linear", "addmm"):
            if name == "addmm":
                b, x, w = specs
                order = [1, 2, 0]
            else:
                x, w = specs[0], specs[1]
                b = specs[2] if len(specs) > 2 else None
                order = [0, 1, 2][:len(specs)]
            w_slot = slots[order[1]]
            if w_slot in self._annotated:
                # a fixed weight layout wins over a derived activation layout: an activation split over the same mesh axis
                # on another dim (sequence parallel in front of a column-parallel product) is gathered first
                taken = {m for m in w.dims_mapping if m != -1}
                k_axis = w.dims_mapping[-1 if name == "linear" else -2] if w.ndim >= 2 else -1
                x = x.with_mapping([-1 if (m in taken and not (d == x.ndim - 1 and m == k_axis)) else m
                                    for d, m in enumerate(x.dims_mapping)])
            new_in, outs = R("matmul").infer_forward(x, w, False, name == "linear")
            new = [None] * len(specs)
            new[order[0]], new[order[1]] = new_in[0], new_in[1]
            if b is not None:
                new[order[2]] = b.with_mapping([outs[0].dims_mapping[-1]] if b.ndim == 1 else [-1] * (b.ndim - 1) + [outs[0].dims_mapping[-1]])
            k = x.shape[-1]
            return "matmul", (new, outs), slots, {"k": k, "x": order[0], "w": order[1]}
        if name == "scaled_dot_product_attention":
            sw = lambda sp: DistTensorSpec([sp.shape[0], sp.shape[2], sp.shape[1], sp.shape[3]],      # noqa: E731
                                           [sp.dims_mapping[0], sp.dims_mapping[2], sp.dims_mapping[1], sp.dims_mapping[3]])
            if all(sp.ndim == 4 for sp in specs[:3]):
                new_in, outs = R("flash_attention").infer_forward(*[sw(sp) for sp in specs[:3]])
                new = [sw(sp) for sp in new_in[:3]] + [sp.with_mapping([-1] * sp.ndim) for sp in specs[3:]]
                causal = bool(node.kwargs.get("is_causal", False))
                return "attention", (new, [sw(outs[0])]), slots, {"causal": causal}
        if name == "embedding":
            new_in, outs = R("embedding").infer_forward(specs[0], specs[1])
            return "embedding", (new_in + [sp.with_mapping([-1] * sp.ndim) for sp in specs[2:]], outs), slots, {}
        if name == "layer_norm":
            x = specs[0]
            nshape = _arg(node, 1, "normalized_shape")
            by = {id(r): sp for r, sp in zip(refs, specs)}
            w, b = _arg(node, 2, "weight"), _arg(node, 3, "bias")
            new_in, outs = R("layer_norm").infer_forward(x, by.get(id(w)), by.get(id(b)), 1e-5, x.ndim - len(nshape))
            return "norm", (new_in, outs[:1]), [refs[0].slot] + [r.slot for r in (w, b) if _is_ref(r)], {}
        if name == "rms_norm":
            x = specs[0]
            w = _arg(node, 2, "weight")
            by = {id(r): sp for r, sp in zip(refs, specs)}
            new_in, outs = R("rms_norm").infer_forward(x, by.get(id(w)))
            return "norm", (new_in, outs[:1]), [refs[0].slot] + ([w.slot] if _is_ref(w) else []), {}
        if name in ("softmax", "log_softmax"):
            new_in, outs = R("softmax").infer_forward(specs[0], _arg(node, 1, "dim", -1))
            return "softmax", (new_in, outs), slots[:1], {}
        if name in ("cross_entropy", "nll_loss") and len(specs) >= 2:
            x, lab = specs[0], specs[1]
            axis = 1 if x.ndim > 1 else 0
            soft = lab.ndim == x.ndim
            lab_r = lab if soft else DistTensorSpec(lab.shape[:axis] + [1] + lab.shape[axis:], lab.dims_mapping[:axis] + [-1] + lab.dims_mapping[axis:])
            new_in, outs = R("cross_entropy_with_softmax").infer_forward(x, lab_r, soft, True, True, -100, axis)
            lab_new = new_in[1] if soft else lab.with_mapping(new_in[1].dims_mapping[:axis] + new_in[1].dims_mapping[axis + 1:])
            loss = outs[1]
            loss_map = loss.dims_mapping[:axis] + loss.dims_mapping[axis + 1:]
            osh = out_shapes[0]
            if len(osh) == len(loss_map):
                out = DistTensorSpec(osh, loss_map)
            else:                                   # reduced inside the call: a partial value over the split sample dims
                out = DistTensorSpec(osh, [-1] * len(osh), {m for m in loss_map if m != -1})
            extra = [sp.with_mapping([-1] * sp.ndim) for sp in specs[2:]]
            return "loss", ([new_in[0], lab_new] + extra, [out]), slots, {"classes": x.shape[axis]}
        if name in _REDUCE and len(specs) == 1:
            dim = _arg(node, 1, "dim", None)
            if isinstance(dim, (int, list, tuple)) or dim is None:
                keep = bool(_arg(node, 2, "keepdim", False))
                rule = "sum" if name in ("sum", "mean", "amax", "amin", "max", "min", "all", "any") else "logsumexp"
                new_in, outs = R(rule).infer_forward(specs[0], dim, keep)
                outs = [outs[0]] + [outs[0].with_mapping(outs[0].dims_mapping) for _ in out_shapes[1:]]
                return "reduce", (new_in, outs), slots, {}
        if name in _LAYOUT_RESHAPE and out_shapes:
            new_in, outs = R("reshape").infer_forward(specs[0], out_shapes[0], self.ctx.mesh_shape)
            return "layout", (new_in + [sp.with_mapping([-1] * sp.ndim) for sp in specs[1:]], outs), slots, {}
        if name in ("permute", "transpose", "t", "swapaxes", "swapdims", "movedim", "__get__"):
            x = specs[0]
            perm = self._perm(node, name, x.ndim)
            if perm is not None:
                new_in, outs = R("transpose").infer_forward(x, perm)
                return "layout", (new_in, outs), slots[:1], {}
            if name == "__get__" and out_shapes and out_shapes[0] == x.shape:      # .data / .real of a real tensor
                return "layout", ([x], [x.with_mapping(x.dims_mapping)]), slots[:1], {}
        if name in ("unsqueeze", "squeeze") and out_shapes:
            new_in, outs = R("reshape").infer_forward(specs[0], out_shapes[0], self.ctx.mesh_shape)
            return "layout", (new_in, outs), slots[:1], {}
        if name in ("cat", "concat", "stack") and isinstance(node.args[0], (list, tuple)):
            dim = _arg(node, 1, "dim", 0)
            new_in, outs = R("stack" if name == "stack" else "concat").infer_forward(specs, dim)
            return "layout", (new_in[0], outs), slots, {}
        if name in ("split", "chunk", "unbind") and len(specs) == 1:
            dim = _arg(node, 2, "dim", 0) if name != "unbind" else _arg(node, 1, "dim", 0)
            x = specs[0]
            d = dim % x.ndim
            m = list(x.dims_mapping)
            m[d] = -1
            om = m if name != "unbind" else m[:d] + m[d + 1:]
            return "layout", ([x.with_mapping(m)], [DistTensorSpec(sh, om) for sh in out_shapes]), slots, {}
        if name in ("__getitem__", "narrow", "select", "slice", "index_select", "gather", "take_along_dim") and out_shapes:
            x = specs[0]
            if len(out_shapes[0]) == x.ndim:
                m = [mm if so == si else -1 for mm, so, si in zip(x.dims_mapping, out_shapes[0], x.shape)]
                ins = [x.with_mapping(m)] + [sp.with_mapping([-1] * sp.ndim) for sp in specs[1:]]
                return "layout", (ins, [DistTensorSpec(out_shapes[0], m)]), slots, {}
        if name in ("conv2d", "conv1d", "conv3d") and len(specs) >= 2 and name == "conv2d":
            new_in, outs = R("conv2d").infer_forward(specs[0], specs[1])
            bias = [sp.with_mapping([outs[0].dims_mapping[1]]) for sp in specs[2:3]]
            return "matmul", (new_in + bias, outs), slots, {"k": specs[1].shape[1] * specs[1].shape[2] * specs[1].shape[3], "x": 0, "w": 1}
        if name in _ELEMENTWISE and out_shapes and all(len(out_shapes[0]) >= sp.ndim for sp in specs):
            new_in, outs = R("elementwise").infer_forward(*specs)
            if outs[0].shape == out_shapes[0]:
                return "elementwise", (new_in, outs + [outs[0].with_mapping(outs[0].dims_mapping) for _ in out_shapes[1:]]), slots, {}
        # no rule: whole inputs, whole outputs
        return "other", ([sp.with_mapping([-1] * sp.ndim) for sp in specs],
                         [DistTensorSpec(sh, [-1] * len(sh)) for sh in out_shapes]), slots, {}

    def _strip(self, sp):
        if not (sp.partial_dims and self.prefer_scatter and self._cur_elementwise):
            return sp
        m = list(sp.dims_mapping)
        for a in sp.partial_dims:
            d = self.prefer_scatter.get(a)
            if d is not None and d < sp.ndim and a not in m and m[d] == -1 and sp.shape[d] % self.ctx.mesh_shape[a] == 0:
                m[d] = a
        return DistTensorSpec(sp.shape, m, sp.partial_dims)

    def _perm(self, node, name, nd):
        if name == "permute":
            dims = node.args[1:] if len(node.args) > 1 else node.kwargs.get("dims", ())
            dims = list(dims[0]) if len(dims) == 1 and isinstance(dims[0], (list, tuple)) else list(dims)
            return [d % nd for d in dims]
        if name in ("transpose", "swapaxes", "swapdims"):
            a, b = _arg(node, 1, "dim0"), _arg(node, 2, "dim1")
            perm = list(range(nd))
            perm[a % nd], perm[b % nd] = perm[b % nd], perm[a % nd]
            return perm
        if name == "t":
            return list(range(nd))[::-1]
        if name == "__get__":
            attr = getattr(getattr(node.func, "__self__", None), "__name__", None)
            how = _ATTR_PERM.get(attr)
            if how == "reverse":
                return list(range(nd))[::-1]
            if how == "last2" and nd >= 2:
                return list(range(nd - 2)) + [nd - 1, nd - 2]
        return None

    # ---------------------------------------------------------------- the pass
    def complete_forward_annotation(self, program=None):
        ctx = self.ctx
        ctx.dist_ops = []
        ctx.tensor_specs = {}
        ms = ctx.mesh_shape
        for node in _flat(self.program._nodes):
            if self.pre_op_hook is not None:
                self.pre_op_hook(self, node)
            for r in _refs((node.args, node.kwargs)):
                self._spec(r.slot)
            kind, (new_in, outs), slots, attrs = self._infer(node)
            op = DistOp(node, node.name, kind, list(slots), [], list(node.out_slots), [], attrs=attrs)
            for s, want in zip(slots, new_in):
                have = self._spec(s)
                want = DistTensorSpec(have.shape, want.dims_mapping)          # what is consumed is never partial
                op.in_specs.append(want)
                if have.dims_mapping != want.dims_mapping or have.partial_dims:
                    rs = self._reshard(s, have, want)
                    if rs is not None:
                        op.reshards.append(rs)
                        if s in ctx.params and s not in self._annotated and not have.partial_dims:
                            # an un-annotated parameter simply lives in the layout its consumer wants
                            ctx.tensor_specs[s] = want
                            op.reshards.pop()
            for s, sp in zip(node.out_slots, outs):
                if s in self._annotated:                                     # a user annotation on an intermediate wins
                    forced = DistTensorSpec(sp.shape, self._annotated[s])
                    rs = self._reshard(s, sp, forced)
                    if rs is not None:
                        op.out_reshards.append(rs)
                    sp = forced
                ctx.tensor_specs[s] = sp
                op.out_specs.append(sp)
            # gradients of parameters: summed over the axes that split the operator's data but not the parameter
            used = set()
            for sp in op.in_specs + op.out_specs:
                used |= {m for m in sp.dims_mapping if m != -1} | set(sp.partial_dims)
            for s, sp in zip(slots, op.in_specs):
                if s in ctx.params:
                    op.param_slots.append(s)
                    axes = sorted(a for a in used if a not in sp.dims_mapping and ms[a] > 1)
                    if axes:
                        op.grad_sync[s] = axes
            self._backward_comm(op)
            ctx.dist_ops.append(op)
        return ctx

    def _backward_comm(self, op):
        """Collectives that only the backward pass of ``op`` needs: the gradient of a matmul's activation input is a
        partial sum over every mesh axis that splits the weight's output dim; it is all-reduced unless the forward
        all-gathered that input over the same axis (then the mirrored reduce-scatter does the sum)."""
        if op.kind != "matmul" or len(op.in_specs) < 2:
            return
        xi, wi = op.attrs.get("x", 0), op.attrs.get("w", 1)
        x, w = op.in_specs[xi], op.in_specs[wi]
        xs = op.in_slots[xi]
        if xs in self.ctx.placeholders.values() or xs in self.ctx.params:
            return
        out = op.out_specs[0]
        n_axis = out.dims_mapping[-1]
        if n_axis == -1 or n_axis in x.dims_mapping:
            return
        gathered = any(r.slot == xs and any(st.kind == "all_gather" and st.mesh_axis == n_axis for st in r.steps) for r in op.reshards)
        if not gathered:
            op.backward_comm.append(CommStep("all_reduce", n_axis, self.ctx.nbytes(xs, x)))
