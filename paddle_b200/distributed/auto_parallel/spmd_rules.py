"""SPMD inference rules (paddle/phi/infermeta/spmd_rules/*.cc, registry in rules.cc; Python access through
``core.get_phi_spmd_rule(name).infer_forward(...)``): given how the inputs of an operator are sharded over the process
mesh, decide how each input has to be sharded for the operator to run on local shards, and how the outputs come out
(sharded, replicated, or partial = pending a reduction over a mesh axis).

A tensor's distribution is a ``dims_mapping``: entry ``i`` is the mesh axis that splits tensor dimension ``i`` or -1.
Most rules are written in einsum notation: every tensor dimension gets a letter, equal letters must be sharded alike,
a mesh axis may split one letter only, and a letter that is sharded in the inputs but absent from the output makes the
output partial on that mesh axis.  The rules are pure functions of shapes and mappings, so they are checked without a
process group; ``dist_tensor._dispatch`` applies them to run operators on ``DistTensor``."""
from __future__ import annotations

import string
from dataclasses import dataclass, field


@dataclass
class DistTensorSpec:
    shape: list
    dims_mapping: list
    partial_dims: set = field(default_factory=set)      # mesh axes on which the value is a partial sum

    def __post_init__(self):
        self.shape, self.dims_mapping = list(self.shape), list(self.dims_mapping)
        self.partial_dims = set(self.partial_dims)
        if len(self.shape) != len(self.dims_mapping):
            raise ValueError(f"dims_mapping {self.dims_mapping} does not match the rank of shape {self.shape}")

    @property
    def ndim(self):
        return len(self.shape)

    def with_mapping(self, dims_mapping, partial_dims=()):
        return DistTensorSpec(self.shape, dims_mapping, partial_dims)

    def is_partial(self):
        return bool(self.partial_dims)


def spec(shape, dims_mapping=None, partial_dims=()):
    return DistTensorSpec(shape, [-1] * len(shape) if dims_mapping is None else dims_mapping, partial_dims)


# ------------------------------------------------------------------------------------------------------ einsum engine
def _merge_letters(axes_list, specs, banned=()):
    """letter -> mesh axis.  The first sharded occurrence of a letter wins; a mesh axis keeps the first letter it
    splits (later letters on the same mesh axis become replicated); size-1 dimensions never count as sharded."""
    letter_to_mesh = {}
    for axes, sp in zip(axes_list, specs):
        for ax, m, size in zip(axes, sp.dims_mapping, sp.shape):
            if ax == "1" or size == 1:
                continue
            if ax in banned:
                letter_to_mesh[ax] = -1
                continue
            if m != -1 and letter_to_mesh.get(ax, -1) == -1:
                letter_to_mesh[ax] = m
            letter_to_mesh.setdefault(ax, -1)
    seen = {}
    for axes in axes_list:
        for ax in axes:
            m = letter_to_mesh.get(ax, -1)
            if m == -1:
                continue
            if m in seen and seen[m] != ax:
                letter_to_mesh[ax] = -1
            else:
                seen[m] = ax
    return letter_to_mesh


def _apply(axes, sp, letter_to_mesh):
    return [(-1 if (ax == "1" or size == 1) else letter_to_mesh.get(ax, -1)) for ax, size in zip(axes, sp.shape)]


def einsum_infer(in_axes, in_specs, out_axes, out_shapes, replicated_letters=(), reduce_letters=None):
    """-> (new input specs, output specs).  ``replicated_letters`` may not be sharded at all; letters of the inputs that
    appear in no output (or are listed in ``reduce_letters``) turn their mesh axis into a partial axis of the outputs."""
    l2m = _merge_letters(in_axes, in_specs, set(replicated_letters))
    new_in = [sp.with_mapping(_apply(axes, sp, l2m)) for axes, sp in zip(in_axes, in_specs)]
    out_letters = set("".join(out_axes))
    reduced = set(reduce_letters) if reduce_letters is not None else {ax for axes in in_axes for ax in axes if ax not in out_letters}
    partial = {l2m[ax] for ax in reduced if l2m.get(ax, -1) != -1}
    outs = []
    for axes, shp in zip(out_axes, out_shapes):
        dm = [(-1 if (ax == "1" or size == 1) else l2m.get(ax, -1)) for ax, size in zip(axes, shp)]
        outs.append(DistTensorSpec(shp, dm, partial))
    return new_in, outs


def _letters(n, skip=""):
    pool = [c for c in string.ascii_lowercase if c not in skip]
    if n > len(pool):
        raise ValueError("tensor rank beyond the notation's alphabet")
    return "".join(pool[:n])


def _broadcast_axes(specs):
    """Right-aligned broadcasting notation: the output takes letters a, b, c ...; an input's size-1 dim becomes '1'."""
    nd = max(s.ndim for s in specs)
    out = _letters(nd)
    out_shape = [1] * nd
    for s in specs:
        for i, size in enumerate(s.shape):
            j = nd - s.ndim + i
            out_shape[j] = max(out_shape[j], size)
    axes = []
    for s in specs:
        off = nd - s.ndim
        axes.append("".join("1" if (size == 1 and out_shape[off + i] != 1) else out[off + i] for i, size in enumerate(s.shape)))
    return axes, out, out_shape


def _norm_axis(axis, nd):
    return axis + nd if axis < 0 else axis


# ------------------------------------------------------------------------------------------------------------- rules
class SpmdRule:
    def __init__(self, name, forward, backward=None):
        self.name, self._fwd, self._bwd = name, forward, backward

    def infer_forward(self, *args, **kwargs):
        return self._fwd(*args, **kwargs)

    def infer_backward(self, *args, **kwargs):
        if self._bwd is None:
            raise NotImplementedError(f"spmd rule {self.name} has no backward inference")
        return self._bwd(*args, **kwargs)


_RULES = {}


def register(*names, backward=None):
    def deco(fn):
        for n in names:
            _RULES[n] = SpmdRule(n, fn, backward)
        return fn
    return deco


def get_phi_spmd_rule(name):
    if name not in _RULES:
        raise KeyError(f"no spmd rule named {name!r}")
    return _RULES[name]


def has_rule(name):
    return name in _RULES


def rule_names():
    return sorted(_RULES)


# --- elementwise family
_UNARY = ("abs", "acos", "acosh", "asin", "asinh", "atan", "atanh", "bitwise_not", "cast", "ceil", "clip", "cos", "cosh", "digamma", "dropout",
          "elu", "erf", "erfinv", "exp", "expm1", "floor", "full_like", "gelu", "hardswish", "leaky_relu", "lgamma", "log", "log10", "log1p",
          "log2", "logical_not", "logit", "neg", "pow", "reciprocal", "relu", "relu6", "round", "rsqrt", "scale", "selu", "sigmoid", "sign",
          "silu", "sin", "sinh", "softplus", "sqrt", "square", "swish", "tan", "tanh", "trunc", "assign", "isfinite", "isnan", "isinf")
_BINARY = ("add", "subtract", "multiply", "divide", "maximum", "minimum", "floor_divide", "remainder", "elementwise_pow", "bitwise_and",
           "bitwise_or", "bitwise_xor", "logical_and", "logical_or", "logical_xor", "equal", "not_equal", "greater_than", "greater_equal",
           "less_than", "less_equal", "fmax", "fmin", "atan2", "heaviside", "copysign")


@register("elementwise", "where", "fused_dropout_add", "add_n_pairwise", *_UNARY, *_BINARY)
def elementwise_rule(*specs_and_attrs):
    specs = [s for s in specs_and_attrs if isinstance(s, DistTensorSpec)]
    axes, out, out_shape = _broadcast_axes(specs)
    new_in, outs = einsum_infer(axes, specs, [out], [out_shape])
    return new_in, outs


def _elementwise_backward(*args):
    *ins, out = [a for a in args if isinstance(a, DistTensorSpec)]
    axes, out_axes, _ = _broadcast_axes(ins)
    l2m = {ax: m for ax, m in zip(out_axes, out.dims_mapping)}
    return [sp.with_mapping(_apply(a, sp, l2m)) for a, sp in zip(axes, ins)], [out.with_mapping(out.dims_mapping)]


for _n in ("elementwise",) + _UNARY + _BINARY:
    _RULES[_n]._bwd = _elementwise_backward


@register("add_n")
def add_n_rule(xs):
    new_in, outs = elementwise_rule(*xs)
    return [new_in], outs


@register("swiglu")
def swiglu_rule(x, y=None):
    if y is not None:
        return elementwise_rule(x, y)
    ax = _letters(x.ndim)
    out_shape = x.shape[:-1] + [x.shape[-1] // 2]
    return einsum_infer([ax], [x], [ax], [out_shape], replicated_letters=ax[-1])


# --- contraction
@register("matmul")
def matmul_rule(x, y, trans_x=False, trans_y=False):
    xn, yn = x.ndim, y.ndim
    if xn == 1 and yn == 1:
        return einsum_infer(["k", "k"], [x, y], [""], [[]])
    batch_n = max(xn, yn) - 2
    batch = _letters(max(batch_n, 0), skip="mnk")
    xa = ("km" if trans_x else "mk") if xn >= 2 else "k"
    ya = ("nk" if trans_y else "kn") if yn >= 2 else "k"
    xb = batch[batch_n - (xn - 2):] if xn > 2 else ""
    yb = batch[batch_n - (yn - 2):] if yn > 2 else ""
    bshape = []
    for i in range(batch_n):
        sx = x.shape[i - (batch_n - (xn - 2))] if xn > 2 and i >= batch_n - (xn - 2) else 1
        sy = y.shape[i - (batch_n - (yn - 2))] if yn > 2 and i >= batch_n - (yn - 2) else 1
        bshape.append(max(sx, sy))
    xfull = "".join("1" if (x.shape[i] == 1 and bshape[batch_n - (xn - 2) + i] != 1) else c for i, c in enumerate(xb)) + xa
    yfull = "".join("1" if (y.shape[i] == 1 and bshape[batch_n - (yn - 2) + i] != 1) else c for i, c in enumerate(yb)) + ya
    m = x.shape[-1 if trans_x else -2] if xn >= 2 else None
    n = y.shape[-2 if trans_y else -1] if yn >= 2 else None
    out_axes = batch + ("m" if m is not None else "") + ("n" if n is not None else "")
    out_shape = bshape + ([m] if m is not None else []) + ([n] if n is not None else [])
    return einsum_infer([xfull, yfull], [x, y], [out_axes], [out_shape])


def _matmul_backward(x, y, out, trans_x=False, trans_y=False):
    """From the output's mapping: batch / m / n letters flow back to the inputs, k stays replicated."""
    new_in, _ = matmul_rule(x.with_mapping([-1] * x.ndim), y.with_mapping([-1] * y.ndim), trans_x, trans_y)
    xn, yn, on = x.ndim, y.ndim, out.ndim
    xm, ym = [-1] * xn, [-1] * yn
    batch_n = on - (1 if xn >= 2 else 0) - (1 if yn >= 2 else 0)
    for i in range(batch_n):
        mi = out.dims_mapping[i]
        xi, yi = i - (batch_n - (xn - 2)), i - (batch_n - (yn - 2))
        if xn > 2 and xi >= 0 and x.shape[xi] != 1:
            xm[xi] = mi
        if yn > 2 and yi >= 0 and y.shape[yi] != 1:
            ym[yi] = mi
    pos = batch_n
    if xn >= 2:
        xm[-1 if trans_x else -2] = out.dims_mapping[pos]
        pos += 1
    if yn >= 2:
        ym[-2 if trans_y else -1] = out.dims_mapping[pos]
    return [x.with_mapping(xm), y.with_mapping(ym)], [out.with_mapping(out.dims_mapping)]


_RULES["matmul"]._bwd = _matmul_backward


@register("fused_linear_param_grad_add")
def fused_linear_param_grad_add_rule(x, dout, dweight=None, dbias=None, multi_precision=True, has_bias=True):
    """dW = x^T dout over all leading dims: shards of the token dims make dW (and dbias) partial."""
    lead = _letters(x.ndim - 1, skip="kn")
    new_in, outs = einsum_infer([lead + "k", lead + "n"], [x, dout], ["kn", "n"], [[x.shape[-1], dout.shape[-1]], [dout.shape[-1]]])
    return new_in, outs if has_bias else outs[:1]


@register("conv2d")
def conv2d_rule(input, filter, strides=(1, 1), paddings=(0, 0), padding_algorithm="EXPLICIT", dilations=(1, 1), groups=1, data_format="NCHW"):
    """Batch and output channels may be split; a split of the input channels makes the output partial; spatial dims stay
    whole.  Grouped convolutions keep the channels whole."""
    if data_format == "NCHW":
        ia, oa = "nchw", "nmHW"
    else:
        ia, oa = "nhwc", "nHWm"
    out_shape = [input.shape[0], filter.shape[0], -1, -1] if data_format == "NCHW" else [input.shape[0], -1, -1, filter.shape[0]]
    no_split = "hwxy" + ("cm" if groups != 1 else "")
    return einsum_infer([ia, "mcxy"], [input, filter], [oa], [out_shape], replicated_letters=no_split)


# --- reductions
def _reduction(x, axis=None, keep_dim=False, partial=True):
    nd = x.ndim
    if axis is None or (isinstance(axis, (list, tuple)) and len(axis) == 0):
        rdims = list(range(nd))
    else:
        rdims = sorted({_norm_axis(a, nd) for a in (axis if isinstance(axis, (list, tuple)) else [axis])})
    ax = _letters(nd)
    if keep_dim:
        out_axes = "".join("1" if i in rdims else c for i, c in enumerate(ax))
        out_shape = [1 if i in rdims else s for i, s in enumerate(x.shape)]
    else:
        out_axes = "".join(c for i, c in enumerate(ax) if i not in rdims)
        out_shape = [s for i, s in enumerate(x.shape) if i not in rdims]
    red = [ax[i] for i in rdims]
    if partial:
        return einsum_infer([ax], [x], [out_axes], [out_shape], reduce_letters=red)
    return einsum_infer([ax], [x], [out_axes], [out_shape], replicated_letters=red, reduce_letters=[])


@register("sum", "mean", "max", "min", "prod", "all", "any", "reduction", "logsumexp", "amax", "amin")
def reduction_rule(x, axis=None, keep_dim=False, *unused):
    """Linear reductions (sum, mean, max, min, all, any) finish with a reduction over the mesh axis: the output is
    partial.  ``prod`` / ``logsumexp`` are not: their reduced dims are gathered first."""
    return _reduction(x, axis, keep_dim)


_RULES["prod"]._fwd = lambda x, axis=None, keep_dim=False, *u: _reduction(x, axis, keep_dim, partial=False)
_RULES["logsumexp"]._fwd = lambda x, axis=None, keep_dim=False, *u: _reduction(x, axis, keep_dim, partial=False)


@register("squared_l2_norm", "numel")
def full_reduction_rule(x):
    return _reduction(x, None, False)


@register("p_norm")
def p_norm_rule(x, porder=2.0, axis=-1, epsilon=1e-12, keepdim=False, asvector=False):
    return _reduction(x, None if asvector else axis, keepdim, partial=False)


@register("argmax", "argmin")
def argmax_rule(x, axis=None, keepdims=False, flatten=False, dtype="int64"):
    if flatten or axis is None:
        return einsum_infer([_letters(x.ndim)], [x], [""], [[]], replicated_letters=_letters(x.ndim), reduce_letters=[])
    return _reduction(x, axis, keepdims, partial=False)


@register("cumsum", "cumprod", "logcumsumexp", "cummax", "cummin")
def cumsum_rule(x, axis=-1, flatten=False, exclusive=False, reverse=False):
    ax = _letters(x.ndim)
    if flatten:
        n = 1
        for s in x.shape:
            n *= s
        return einsum_infer([ax], [x], ["z"], [[n]], replicated_letters=ax, reduce_letters=[])
    return einsum_infer([ax], [x], [ax], [x.shape], replicated_letters=ax[_norm_axis(axis, x.ndim)])


# --- normalisation / softmax
@register("softmax", "log_softmax")
def softmax_rule(x, axis=-1):
    ax = _letters(x.ndim)
    return einsum_infer([ax], [x], [ax], [x.shape], replicated_letters=ax[_norm_axis(axis, x.ndim)])


@register("layer_norm")
def layer_norm_rule(x, scale=None, bias=None, epsilon=1e-5, begin_norm_axis=1):
    """Dims from ``begin_norm_axis`` on are normalised together and stay whole; scale / bias are replicated;
    outputs: y, mean, variance (the latter two over the leading dims)."""
    ax = _letters(x.ndim)
    b = _norm_axis(begin_norm_axis, x.ndim)
    ins, in_axes = [x], [ax]
    n = 1
    for s in x.shape[b:]:
        n *= s
    for t in (scale, bias):
        if t is not None:
            ins.append(t)
            in_axes.append("z")
    new_in, outs = einsum_infer(in_axes, ins, [ax, ax[:b], ax[:b]], [x.shape, x.shape[:b], x.shape[:b]], replicated_letters=ax[b:] + "z",
                                reduce_letters=[])
    return new_in, outs


@register("rms_norm")
def rms_norm_rule(x, scale=None, epsilon=1e-6):
    ax = _letters(x.ndim)
    ins, in_axes = [x], [ax]
    if scale is not None:
        ins.append(scale)
        in_axes.append(ax[-1])
    return einsum_infer(in_axes, ins, [ax, ax[:-1]], [x.shape, x.shape[:-1]], replicated_letters=ax[-1], reduce_letters=[])


# --- embedding / losses
@register("embedding", "c_embedding")
def embedding_rule(x, weight, padding_idx=-1, sparse=False):
    """Row (vocabulary) shards of the table give a partial output (each rank contributes the rows it owns); column shards
    split the last output dim; index dims pass through."""
    ia = _letters(x.ndim, skip="vh")
    out_shape = x.shape + [weight.shape[1]]
    return einsum_infer([ia, "vh"], [x, weight], [ia + "h"], [out_shape], reduce_letters=["v"])


@register("cross_entropy_with_softmax", "c_softmax_with_cross_entropy")
def cross_entropy_with_softmax_rule(x, label, soft_label=False, use_softmax=True, numeric_stable_mode=True, ignore_index=-100, axis=-1):
    """-> (softmax_out, loss).  The class dim may stay sharded (the vocab-parallel form: maxima and sums are reduced over
    that mesh axis inside the operator), the loss has size 1 there; every other dim passes through."""
    nd = x.ndim
    a = _norm_axis(axis, nd)
    ax = _letters(nd)
    lab_axes = ax if soft_label else "".join("1" if i == a else c for i, c in enumerate(ax))
    loss_axes = "".join("1" if i == a else c for i, c in enumerate(ax))
    loss_shape = [1 if i == a else s for i, s in enumerate(x.shape)]
    new_in, outs = einsum_infer([ax, lab_axes], [x, label], [ax, loss_axes], [x.shape, loss_shape], reduce_letters=[])
    return new_in, outs


# --- layout
@register("transpose")
def transpose_rule(x, perm):
    ax = _letters(x.ndim)
    perm = [_norm_axis(p, x.ndim) for p in perm]
    return einsum_infer([ax], [x], ["".join(ax[p] for p in perm)], [[x.shape[p] for p in perm]])


def _dim_groups(src, dst):
    """Split two shapes with equal products into aligned groups: [(src dims, dst dims)] with equal products each."""
    groups, i, j = [], 0, 0
    while i < len(src) or j < len(dst):
        si, dj = [i] if i < len(src) else [], [j] if j < len(dst) else []
        ps = src[i] if i < len(src) else 1
        pd = dst[j] if j < len(dst) else 1
        i, j = i + (1 if si else 0), j + (1 if dj else 0)
        while ps != pd:
            if ps < pd:
                ps *= src[i]
                si.append(i)
                i += 1
            else:
                pd *= dst[j]
                dj.append(j)
                j += 1
        groups.append((si, dj))
    return groups


@register("reshape", "flatten", "view")
def reshape_rule(x, shape, mesh_shape=None):
    """A sharded source dim keeps its shard when it is the leading dim of its group (flatten: leading factor of the merged
    dim; split: leading piece) and - with ``mesh_shape`` given - the destination's leading dim divides by the size of that
    mesh axis; other sharded dims are gathered."""
    numel = 1
    for s in x.shape:
        numel *= s
    shape = [x.shape[i] if s == 0 else s for i, s in enumerate(shape)]          # 0 copies the source dim
    if -1 in shape:
        known = 1
        for s in shape:
            known *= s if s != -1 else 1
        shape[shape.index(-1)] = numel // max(known, 1)
    in_map = list(x.dims_mapping)
    out_map = [-1] * len(shape)
    for sg, dg in _dim_groups(x.shape, shape):
        sg_real = [i for i in sg if x.shape[i] != 1] or sg
        dg_real = [j for j in dg if shape[j] != 1] or dg
        for i in sg:
            if in_map[i] != -1 and (not sg_real or i != sg_real[0] or not dg_real):
                in_map[i] = -1
        if sg_real and dg_real and in_map[sg_real[0]] != -1:
            m = in_map[sg_real[0]]
            same_dim = len(sg_real) == 1 and len(dg_real) == 1            # the dim is carried over unchanged
            if not same_dim and mesh_shape is not None and shape[dg_real[0]] % mesh_shape[m]:
                in_map[sg_real[0]] = -1
            else:
                out_map[dg_real[0]] = m
    return [x.with_mapping(in_map)], [DistTensorSpec(shape, out_map)]


@register("squeeze")
def squeeze_rule(x, axis=None):
    nd = x.ndim
    axes = [i for i, s in enumerate(x.shape) if s == 1] if axis is None or axis == [] else \
        [_norm_axis(a, nd) for a in (axis if isinstance(axis, (list, tuple)) else [axis]) if x.shape[_norm_axis(a, nd)] == 1]
    keep = [i for i in range(nd) if i not in axes]
    ax = _letters(nd)
    return einsum_infer([ax], [x], ["".join(ax[i] for i in keep)], [[x.shape[i] for i in keep]])


@register("unsqueeze")
def unsqueeze_rule(x, axis):
    axes = sorted(_norm_axis(a, x.ndim + len(axis if isinstance(axis, (list, tuple)) else [axis])) for a in
                  (axis if isinstance(axis, (list, tuple)) else [axis]))
    ax = list(_letters(x.ndim))
    shape = list(x.shape)
    for a in axes:
        ax.insert(a, "1")
        shape.insert(a, 1)
    return einsum_infer([_letters(x.ndim)], [x], ["".join(ax)], [shape])


@register("concat")
def concat_rule(xs, axis=0):
    nd = xs[0].ndim
    a = _norm_axis(axis, nd)
    ax = _letters(nd)
    out_shape = list(xs[0].shape)
    out_shape[a] = sum(t.shape[a] for t in xs)
    new_in, outs = einsum_infer([ax] * len(xs), xs, [ax], [out_shape], replicated_letters=ax[a])
    return [new_in], outs


@register("stack")
def stack_rule(xs, axis=0):
    nd = xs[0].ndim
    a = _norm_axis(axis, nd + 1)
    ax = _letters(nd)
    out_axes = ax[:a] + "1" + ax[a:]
    out_shape = xs[0].shape[:a] + [len(xs)] + xs[0].shape[a:]
    new_in, outs = einsum_infer([ax] * len(xs), xs, [out_axes], [out_shape])
    return [new_in], outs


@register("split", "split_with_num", "chunk")
def split_rule(x, sections, axis=0):
    nd = x.ndim
    a = _norm_axis(axis, nd)
    sizes = [x.shape[a] // sections] * sections if isinstance(sections, int) else list(sections)
    if -1 in sizes:
        sizes[sizes.index(-1)] = x.shape[a] - sum(s for s in sizes if s != -1)
    ax = _letters(nd)
    shapes = [x.shape[:a] + [s] + x.shape[a + 1:] for s in sizes]
    new_in, outs = einsum_infer([ax], [x], [ax] * len(sizes), shapes, replicated_letters=ax[a])
    return new_in, [outs]


@register("unbind")
def unbind_rule(x, axis=0):
    nd = x.ndim
    a = _norm_axis(axis, nd)
    ax = _letters(nd)
    out_axes = ax[:a] + ax[a + 1:]
    shp = x.shape[:a] + x.shape[a + 1:]
    new_in, outs = einsum_infer([ax], [x], [out_axes] * x.shape[a], [shp] * x.shape[a], replicated_letters=ax[a], reduce_letters=[])
    return new_in, [outs]


@register("slice", "strided_slice")
def slice_rule(x, axes, starts, ends, infer_flags=None, decrease_axis=()):
    nd = x.ndim
    axes = [_norm_axis(a, nd) for a in axes]
    ax = _letters(nd)
    shape = list(x.shape)
    for a, s, e in zip(axes, starts, ends):
        n = x.shape[a]
        s = max(s + n, 0) if s < 0 else min(s, n)
        e = max(e + n, 0) if e < 0 else min(e, n)
        shape[a] = max(e - s, 0)
    dec = {_norm_axis(a, nd) for a in decrease_axis}
    out_axes = "".join(c for i, c in enumerate(ax) if i not in dec)
    out_shape = [s for i, s in enumerate(shape) if i not in dec]
    return einsum_infer([ax], [x], [out_axes], [out_shape], replicated_letters="".join(ax[a] for a in axes), reduce_letters=[])


@register("tile")
def tile_rule(x, repeat_times):
    reps = list(repeat_times)
    nd = max(x.ndim, len(reps))
    reps = [1] * (nd - len(reps)) + reps
    shape = [1] * (nd - x.ndim) + x.shape
    out = _letters(nd)
    in_axes = out[nd - x.ndim:]
    rep_letters = "".join(out[i] for i in range(nd) if reps[i] != 1)
    return einsum_infer([in_axes], [x], [out], [[s * r for s, r in zip(shape, reps)]], replicated_letters=rep_letters, reduce_letters=[])


@register("expand_as", "expand", "broadcast_to")
def expand_as_rule(x, y=None, target_shape=None):
    shape = list(target_shape if target_shape is not None else y.shape)
    nd = len(shape)
    out = _letters(nd)
    off = nd - x.ndim
    in_axes = "".join("1" if (s == 1 and shape[off + i] != 1) else out[off + i] for i, s in enumerate(x.shape))
    new_in, outs = einsum_infer([in_axes], [x], [out], [shape], reduce_letters=[])
    if y is not None:
        new_in.append(y.with_mapping(outs[0].dims_mapping))
    return new_in, outs


@register("pad")
def pad_rule(x, paddings, pad_value=0.0):
    nd = x.ndim
    ax = _letters(nd)
    pads = list(paddings)
    padded = [i for i in range(nd) if 2 * i + 1 < len(pads) and (pads[2 * i] or pads[2 * i + 1])]
    shape = [s + (pads[2 * i] + pads[2 * i + 1] if 2 * i + 1 < len(pads) else 0) for i, s in enumerate(x.shape)]
    return einsum_infer([ax], [x], [ax], [shape], replicated_letters="".join(ax[i] for i in padded))


@register("triu", "tril")
def triu_rule(x, diagonal=0):
    ax = _letters(x.ndim)
    return einsum_infer([ax], [x], [ax], [x.shape], replicated_letters=ax[-2:])


@register("one_hot")
def one_hot_rule(x, num_classes):
    ax = _letters(x.ndim, skip="z")
    return einsum_infer([ax], [x], [ax + "z"], [x.shape + [int(num_classes)]])


@register("nonzero", "replicated", "unique", "masked_select")
def replicated_rule(*specs_and_attrs):
    """Operators whose output layout depends on the data: every input is gathered, outputs are replicated (their shapes
    are not known to the rule)."""
    ins = [s.with_mapping([-1] * s.ndim) for s in specs_and_attrs if isinstance(s, DistTensorSpec)]
    return ins, []


@register("default_data_parallel")
def default_data_parallel_rule(*specs, mesh_axis=0):
    """Every tensor is split along its dim 0 on one mesh axis (the first that any input already uses there, else 0)."""
    ins = [s for s in specs if isinstance(s, DistTensorSpec)]
    m = next((s.dims_mapping[0] for s in ins if s.ndim and s.dims_mapping[0] != -1), mesh_axis)
    return [s.with_mapping([m] + [-1] * (s.ndim - 1) if s.ndim and s.shape[0] != 1 else [-1] * s.ndim) for s in ins], []


# --- indexing
@register("gather", "index_select", "take_along_axis")
def gather_rule(x, index, axis=0):
    """The gathered dim of ``x`` stays whole; ``index`` (1-D) keeps its shard, which becomes the shard of that output dim;
    the other dims of ``x`` pass through."""
    nd = x.ndim
    a = _norm_axis(axis, nd)
    ax = _letters(nd, skip="z")
    idx_axes = "z" if index.ndim == 1 else ""
    out_axes = ax[:a] + idx_axes + ax[a + 1:]
    out_shape = x.shape[:a] + (list(index.shape) if index.ndim == 1 else []) + x.shape[a + 1:]
    return einsum_infer([ax, idx_axes], [x, index], [out_axes], [out_shape], replicated_letters=ax[a], reduce_letters=[])


@register("gather_nd")
def gather_nd_rule(x, index):
    """Index leading dims pass through; the indexed leading dims of ``x`` stay whole, the trailing ones pass through."""
    k = index.shape[-1]
    ia = _letters(index.ndim - 1, skip="xyzuvw") + "1"
    xa = "".join("xyzuvw"[i] if i < k else c for i, c in enumerate(_letters(x.ndim, skip="xyzuvw" + ia)))
    out_axes = ia[:-1] + xa[k:]
    out_shape = index.shape[:-1] + x.shape[k:]
    return einsum_infer([xa, ia], [x, index], [out_axes], [out_shape], replicated_letters=xa[:k], reduce_letters=[])


@register("scatter", "put_along_axis", "index_add", "scatter_nd_add")
def scatter_rule(x, index, updates, overwrite=True):
    """Dim 0 (the scattered one) stays whole in ``x`` and ``updates``; ``index`` is gathered; trailing dims pass through."""
    ax = _letters(x.ndim, skip="z")
    ua = "z" + ax[1:] if updates.ndim == x.ndim else ax[1:]
    new_in, outs = einsum_infer([ax, "z" if index.ndim == 1 else "", ua], [x, index, updates], [ax], [x.shape],
                                replicated_letters=ax[0] + "z", reduce_letters=[])
    return new_in, outs


# --- transformer blocks
@register("flash_attention", "flash_attn", "scaled_dot_product_attention")
def flash_attention_rule(q, k, v, attn_mask=None, dropout=0.0, causal=False, *unused):
    """[batch, seq, heads, head_dim]: batch and heads may be split (data / tensor parallelism); sequence and head_dim stay
    whole inside one call (sequence parallel attention goes through the context-parallel wrappers).  Grouped-query
    attention: k / v heads follow q's head split only when the group count divides evenly, which the caller checks.
    -> (out, softmax_lse [batch, heads, seq])."""
    ins, axes = [q, k, v], ["bshd", "bthd", "bthd"]
    if k.shape[2] != q.shape[2]:
        axes[1] = axes[2] = "btgd"                       # separate head letter: merged below by hand
    if attn_mask is not None:
        ins.append(attn_mask)
        axes.append("".join(c if s != 1 else "1" for c, s in zip("bhst"[-attn_mask.ndim:], attn_mask.shape)))
    new_in, outs = einsum_infer(axes, ins, ["bshd", "bhs"], [q.shape, [q.shape[0], q.shape[2], q.shape[1]]], replicated_letters="std",
                                reduce_letters=[])
    if k.shape[2] != q.shape[2]:
        hm = new_in[0].dims_mapping[2]
        for t in new_in[1:3]:
            t.dims_mapping[2] = hm
    return new_in, outs


@register("fused_rope", "fused_rotary_position_embedding")
def fused_rope_rule(q, k=None, v=None, sin=None, cos=None, position_ids=None, use_neox_rotary_style=True, time_major=False, rotary_emb_base=10000.0):
    """q / k / v [batch, seq, heads, head_dim] rotate pairs inside head_dim, which stays whole; sin / cos [1, seq, 1,
    head_dim] follow the sequence split; position_ids [batch, seq]."""
    ins, axes = [], []
    for t in (q, k, v):
        if t is not None:
            ins.append(t)
            axes.append("sbhd" if time_major else "bshd")
    n_qkv = len(ins)
    for t in (sin, cos):
        if t is not None:
            ins.append(t)
            axes.append("1s1d" if t.ndim == 4 else "sd")
    if position_ids is not None:
        ins.append(position_ids)
        axes.append("bs")
    new_in, outs = einsum_infer(axes, ins, axes[:n_qkv], [t.shape for t in ins[:n_qkv]], replicated_letters="d", reduce_letters=[])
    return new_in, outs


@register("optimizer", "adam", "adamw", "sgd", "momentum")
def optimizer_rule(param, grad, *states):
    """Parameter, gradient and every same-shaped state share the parameter's layout (a partial gradient is reduced
    first); scalar states (learning rate, beta powers) are replicated.  Outputs mirror the inputs that are updated."""
    m = list(param.dims_mapping)
    if all(x == -1 for x in m):
        m = list(grad.dims_mapping)
    ins = [param.with_mapping(m), grad.with_mapping(m)]
    for s in states:
        if isinstance(s, DistTensorSpec):
            ins.append(s.with_mapping(m if s.shape == param.shape else [-1] * s.ndim))
    outs = [t.with_mapping(t.dims_mapping) for i, t in enumerate(ins) if i != 1]
    return ins, outs


@register("check_finite_and_unscale", "update_loss_scaling", "amp_ops")
def amp_ops_rule(xs, scale, *rest):
    """Gradients keep their layouts; ``found_inf`` is partial (logical or) over every mesh axis that splits a gradient."""
    used = {m for t in xs for m in t.dims_mapping if m != -1}
    return [[t.with_mapping(t.dims_mapping) for t in xs], scale.with_mapping([-1] * scale.ndim)], \
        [[t.with_mapping(t.dims_mapping) for t in xs], DistTensorSpec([1], [-1], used)]


@register("moe_gate_dispatch")
def moe_gate_dispatch_rule(x, gate_logits, k, capacity, use_pad=True):
    """Tokens [s, h] and gate logits [s, e] share the token split; the dispatched buffer [e, capacity, h] is built per
    token shard (so it is partial over that mesh axis when tokens are split)."""
    new_in, outs = einsum_infer(["sh", "se"], [x, gate_logits], ["ech"], [[gate_logits.shape[1], capacity, x.shape[1]]], replicated_letters="e")
    return new_in, outs


@register("moe_combine")
def moe_combine_rule(x, combine_weights, scatter_index):
    """x [s * k, h], weights / index [s, k]: the token split passes to the output [s, h]."""
    new_in, outs = einsum_infer(["th", "sk", "sk"], [x, combine_weights, scatter_index], ["sh"],
                                [[combine_weights.shape[0], x.shape[1]]], replicated_letters="tk", reduce_letters=[])
    return new_in, outs
