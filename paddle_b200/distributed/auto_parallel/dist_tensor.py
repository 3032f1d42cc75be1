"""Distributed tensors: a local shard plus (mesh, placements) and the SPMD dispatch of operators on them
(paddle/phi/core/distributed/auto_parallel/dist_tensor.h; reshard functions in
paddle/phi/core/distributed/auto_parallel/reshard/*.cc: r_to_s, s_to_r, p_to_r, p_to_s, s_to_s, r_to_p;
SPMD rules in paddle/phi/infermeta/spmd_rules/).

Conventions that make plain autograd on the local shards correct:
  * the gradient of a Replicate tensor is the full gradient, identical on every rank of the axis;
  * the gradient of a Shard tensor is the matching shard; the gradient of a Partial tensor is the full gradient.
Every communication step is an autograd function whose backward is its dual (all-gather <-> slice,
reduce-scatter <-> all-gather, all-reduce <-> identity), and whenever an operator consumes an input that is
replicated along a mesh axis on which its output is NOT replicated, that input passes through an
identity-forward / all-reduce-backward node (the ``c_identity`` of tensor parallelism, the gradient all-reduce of
data parallelism).
"""
from __future__ import annotations

import ctypes

import torch

from ..._core.tensor import Tensor
from .. import collective as C
from .process_mesh import Partial, Placement, ProcessMesh, ReduceType, Replicate, Shard


def _plain(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) and type(t) is not torch.Tensor else t


# ----------------------------------------------------------------------------------------- communication nodes
def _gather_cat(x, group, dim):
    n = group.nranks
    x = x.contiguous()
    parts = [torch.empty_like(x) for _ in range(n)]
    C.all_gather(parts, x, group=group)
    return torch.cat([_plain(p) for p in parts], dim=dim)


def _my_chunk(x, group, dim):
    n, r = group.nranks, group.get_group_rank(C.get_rank())
    assert x.shape[dim] % n == 0, f"dim {dim} of size {x.shape[dim]} is not divisible by the mesh axis size {n}"
    return x.chunk(n, dim=dim)[r].contiguous()


def _reduce_scatter(x, group, dim):
    n = group.nranks
    assert x.shape[dim] % n == 0
    chunks = [c.contiguous() for c in x.chunk(n, dim=dim)]
    out = torch.empty_like(chunks[0])
    C.reduce_scatter(out, chunks, group=group)
    return _plain(out)


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _gather_cat(x, group, dim)

    @staticmethod
    def backward(ctx, g):
        return _my_chunk(g, ctx.group, ctx.dim), None, None


class _Slice(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _my_chunk(x, group, dim)

    @staticmethod
    def backward(ctx, g):
        return _gather_cat(g, ctx.group, ctx.dim), None, None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, avg):
        ctx.scale = 1.0 / group.nranks if avg else 1.0
        y = x.contiguous().clone()
        C.all_reduce(y, group=group)
        return _plain(y) * ctx.scale if avg else _plain(y)

    @staticmethod
    def backward(ctx, g):
        return (g * ctx.scale if ctx.scale != 1.0 else g), None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim, avg):
        ctx.group, ctx.dim = group, dim
        ctx.scale = 1.0 / group.nranks if avg else 1.0
        y = _reduce_scatter(x, group, dim)
        return y * ctx.scale if avg else y

    @staticmethod
    def backward(ctx, g):
        full = _gather_cat(g, ctx.group, ctx.dim)
        return (full * ctx.scale if ctx.scale != 1.0 else full), None, None, None


class _AllToAll(torch.autograd.Function):
    """Shard(src_dim) -> Shard(dst_dim) along one axis."""

    @staticmethod
    def forward(ctx, x, group, src_dim, dst_dim):
        ctx.group, ctx.src, ctx.dst = group, src_dim, dst_dim
        return _AllToAll._run(x, group, src_dim, dst_dim)

    @staticmethod
    def _run(x, group, src_dim, dst_dim):
        n = group.nranks
        assert x.shape[dst_dim] % n == 0
        ins = [c.contiguous() for c in x.chunk(n, dim=dst_dim)]
        outs = [torch.empty_like(ins[0]) for _ in range(n)]
        C._alltoall_io(ins, outs, group=group)
        return torch.cat([_plain(o) for o in outs], dim=src_dim)

    @staticmethod
    def backward(ctx, g):
        return _AllToAll._run(g, ctx.group, ctx.dst, ctx.src), None, None, None


class _ToPartial(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        return x if group.get_group_rank(C.get_rank()) == 0 else torch.zeros_like(x)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _IdentityAllReduceBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        C.all_reduce(g, group=ctx.group)
        return _plain(g), None


# ----------------------------------------------------------------------------------------- DistTensor
def _code(p):
    return -1 if p.is_replicated() else (-2 if p.is_partial() else p.dim)


def _global_shape(local_shape, mesh, placements):
    shape = list(local_shape)
    for a, p in enumerate(placements):
        if p.is_shard():
            shape[p.dim] *= mesh.shape[a]
    return shape


def _local_shape(global_shape, mesh, placements):
    shape = list(global_shape)
    for a, p in enumerate(placements):
        if p.is_shard():
            assert shape[p.dim] % mesh.shape[a] == 0, \
                f"global dim {p.dim} ({shape[p.dim]}) is not divisible by mesh axis {a} ({mesh.shape[a]})"
            shape[p.dim] //= mesh.shape[a]
    return shape


def _norm_placements(mesh, placements):
    pl = list(placements or [])
    pl += [Replicate()] * (mesh.ndim - len(pl))
    return pl


class DistTensor(Tensor):
    """The tensor data IS the local shard; ``shape`` reports the global shape like the reference does."""

    @staticmethod
    def wrap(local, mesh, placements, param_like=None):
        t = local if type(local) is DistTensor else local.as_subclass(DistTensor)
        t._dist_mesh = mesh
        t._dist_placements = _norm_placements(mesh, placements)
        return t

    process_mesh = property(lambda self: self._dist_mesh)
    placements = property(lambda self: list(self._dist_placements))

    def is_dist(self):
        return True

    @property
    def shape(self):
        return _global_shape(torch.Tensor.shape.__get__(self), self._dist_mesh, self._dist_placements)

    @property
    def _local_shape(self):
        return list(torch.Tensor.shape.__get__(self))

    def _local_value(self):
        with torch._C.DisableTorchFunctionSubclass():
            return self.as_subclass(Tensor)

    def backward(self, grad_tensor=None, retain_graph=False):
        """Partial values are reduced first, so that each partial contribution receives its share of the
        gradient (1/n for an average) through the reduction's backward."""
        t = self
        if any(p.is_partial() for p in self._dist_placements):
            t = reshard(self, self._dist_mesh, [Replicate() if p.is_partial() else p for p in self._dist_placements])
        g = local_of(grad_tensor) if is_dist(grad_tensor) else grad_tensor
        torch.Tensor.backward(local_of(t), g, retain_graph=retain_graph)

    def dist_attr(self):
        return {"process_mesh": self._dist_mesh, "placements": self.placements}

    def __repr__(self):
        with torch._C.DisableTorchFunctionSubclass():
            body = repr(self.as_subclass(torch.Tensor))
        return f"DistTensor(global_shape={self.shape}, placements={self._dist_placements}, local={body})"

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        return _dispatch(func, args, kwargs or {})


def is_dist(t):
    return isinstance(t, DistTensor)


def local_of(t):
    """Plain torch view of the local shard (keeps the autograd graph)."""
    with torch._C.DisableTorchFunctionSubclass():
        return t.as_subclass(torch.Tensor)


# ----------------------------------------------------------------------------------------- reshard
def _plan(src, dst):
    from ...ops import _lib
    n = len(src)
    a = (ctypes.c_int * n)(*[_code(p) for p in src])
    b = (ctypes.c_int * n)(*[_code(p) for p in dst])
    out = (ctypes.c_int * (3 * 4 * n + 3))()
    steps = _lib.runtime().pd_plan_reshard(a, b, ctypes.c_int(n), out, ctypes.c_int(4 * n + 1))
    return [(out[3 * i], out[3 * i + 1], out[3 * i + 2]) for i in range(steps)]


def reshard_local(x, mesh, src, dst):
    """Apply the planned communication steps to a plain local tensor; returns the new local tensor."""
    src, dst = _norm_placements(mesh, src), _norm_placements(mesh, dst)
    if mesh.coord_of(C.get_rank()) is None:
        return x
    for op, axis, dim in _plan(src, dst):
        g = mesh.get_group(axis)
        if g is None or g.nranks == 1:
            continue
        avg = src[axis].is_partial() and src[axis].reduce_type == ReduceType.kRedAvg
        if op == 1:
            x = _AllGather.apply(x, g, dim)
        elif op == 2:
            x = _AllReduce.apply(x, g, avg)
        elif op == 3:
            x = _ReduceScatter.apply(x, g, dim, avg)
        elif op == 4:
            x = _Slice.apply(x, g, dim)
        elif op == 5:
            x = _AllToAll.apply(x, g, dim // 1000, dim % 1000)
        elif op == 6:
            x = _ToPartial.apply(x, g)
    return x


def reshard(t, mesh, placements):
    placements = _norm_placements(mesh, placements)
    if not is_dist(t):
        from .api import shard_tensor
        return shard_tensor(t, mesh, placements)
    if t._dist_mesh == mesh:
        if t._dist_placements == placements:
            return t
        out = reshard_local(local_of(t), mesh, t._dist_placements, placements)
        return DistTensor.wrap(out, mesh, placements)
    return _cross_mesh(t, mesh, placements)


def _cross_mesh(t, mesh, placements):
    """Same-shape meshes over different ranks (pipeline hand-off, same_status reshard): rank i of the source
    sends its shard to rank i of the destination, then the destination reshards locally."""
    src_mesh = t._dist_mesh
    assert src_mesh.shape == mesh.shape, "cross-mesh reshard needs meshes of the same shape"
    me = C.get_rank()
    x = local_of(t).detach().contiguous()
    out = None
    for s, d in zip(src_mesh.process_ids, mesh.process_ids):
        if s == d:
            if me == s:
                out = x
        elif me == s:
            C.send(x, d)
        elif me == d:
            out = torch.empty(_local_shape(t.shape, mesh, t._dist_placements), dtype=x.dtype, device=x.device)
            C.recv(out, s)
            out = _plain(out)
    if out is None:
        out = torch.empty(0, dtype=x.dtype, device=x.device)
        return DistTensor.wrap(out, mesh, t._dist_placements)
    out = reshard_local(out, mesh, t._dist_placements, placements)
    return DistTensor.wrap(out, mesh, placements)


# ----------------------------------------------------------------------------------------- dispatch
_ELEMENTWISE = {
    "add", "sub", "mul", "div", "true_divide", "pow", "maximum", "minimum", "neg", "abs", "exp", "log", "sqrt", "rsqrt",
    "tanh", "sigmoid", "relu", "gelu", "silu", "square", "sin", "cos", "erf", "clamp", "clip", "where", "eq", "ne", "lt",
    "le", "gt", "ge", "logical_and", "logical_or", "logical_not", "to", "type_as", "float", "half", "bfloat16", "clone",
    "contiguous", "detach", "dropout", "masked_fill", "__add__", "__radd__", "__sub__", "__rsub__", "__mul__", "__rmul__",
    "__truediv__", "__rtruediv__", "__neg__", "__pow__", "leaky_relu", "softplus", "elu", "hardtanh", "floor", "ceil",
    "round", "sign", "reciprocal", "isnan", "isinf", "isfinite", "fmod", "remainder", "add_", "mul_", "sub_", "div_",
    "zero_", "fill_", "copy_", "zeros_like", "ones_like", "empty_like", "full_like", "rand_like", "randn_like", "log1p",
    "expm1", "__eq__", "__ne__", "__lt__", "__le__", "__gt__", "__ge__", "int", "long", "bool", "double", "addcmul",
}
_ROWWISE = {"softmax", "log_softmax", "layer_norm", "rms_norm", "normalize"}
_REDUCE = {"sum", "mean"}
_META = {"size", "dim", "numel", "is_floating_point", "is_contiguous", "stride", "data_ptr", "element_size", "type",
         "get_device", "is_complex", "storage_offset", "untyped_storage", "requires_grad_", "retain_grad", "backward",
         "register_hook", "register_post_accumulate_grad_hook", "__hash__", "__len__", "dim_order", "is_cuda", "nelement",
         "ndimension", "__format__", "__deepcopy__", "__reduce_ex__", "is_shared", "is_pinned", "is_set_to"}


def _flat_tensors(obj, out):
    if isinstance(obj, torch.Tensor):
        out.append(obj)
    elif isinstance(obj, (list, tuple)):
        for o in obj:
            _flat_tensors(o, out)
    elif isinstance(obj, dict):
        for o in obj.values():
            _flat_tensors(o, out)
    return out


def _map_tensors(obj, fn):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, (list, tuple)):
        return type(obj)(_map_tensors(o, fn) for o in obj)
    if isinstance(obj, dict):
        return {k: _map_tensors(v, fn) for k, v in obj.items()}
    return obj


def _run_local(func, args, kwargs):
    with torch._C.DisableTorchFunctionSubclass():
        return func(*_map_tensors(args, lambda t: local_of(t) if is_dist(t) else _plain(t)),
                    **_map_tensors(kwargs, lambda t: local_of(t) if is_dist(t) else _plain(t)))


def _wrap_out(out, mesh, placements):
    def w(t):
        return DistTensor.wrap(t, mesh, placements)
    return _map_tensors(out, w)


def _guard_replicated_inputs(local, mesh, in_pl, out_pl):
    """Identity-forward / all-reduce-backward along every axis where the input is replicated but the output
    differs from rank to rank."""
    if not (isinstance(local, torch.Tensor) and local.requires_grad and torch.is_grad_enabled()):
        return local
    for a in range(mesh.ndim):
        if in_pl[a].is_replicated() and not out_pl[a].is_replicated():
            g = mesh.get_group(a)
            if g is not None and g.nranks > 1:
                local = _IdentityAllReduceBwd.apply(local, g)
    return local


def _to_replicated(t, mesh):
    return reshard(t, mesh, [Replicate()] * mesh.ndim)


def _fallback(func, args, kwargs, mesh):
    """Gather every distributed input, compute replicated."""
    rep = [Replicate()] * mesh.ndim
    conv = lambda t: _to_replicated(t, mesh) if is_dist(t) else t   # noqa: E731
    args, kwargs = _map_tensors(args, conv), _map_tensors(kwargs, conv)
    return _wrap_out(_run_local(func, args, kwargs), mesh, rep)


def _elementwise(func, args, kwargs, mesh, tensors):
    dts = [t for t in tensors if is_dist(t)]
    out_ndim = max(len(t.shape) if is_dist(t) else t.dim() for t in tensors)
    out_pl = [Replicate()] * mesh.ndim
    for a in range(mesh.ndim):
        for t in dts:
            p = t._dist_placements[a]
            if p.is_shard():
                d = p.dim + (out_ndim - len(t.shape))
                if out_pl[a].is_shard() and out_pl[a].dim != d:
                    return _fallback(func, args, kwargs, mesh)
                out_pl[a] = Shard(d)
    used = [p.dim for p in out_pl if p.is_shard()]
    if len(used) != len(set(used)):
        return _fallback(func, args, kwargs, mesh)

    def conv(t):
        nd = len(t.shape) if is_dist(t) else t.dim()
        gshape = t.shape if is_dist(t) else list(t.shape)
        want = []
        for a in range(mesh.ndim):
            p = out_pl[a]
            d = p.dim - (out_ndim - nd) if p.is_shard() else -1
            want.append(Shard(d) if (p.is_shard() and d >= 0 and gshape[d] > 1) else Replicate())
        if not is_dist(t):
            t = DistTensor.wrap(_plain(t), mesh, [Replicate()] * mesh.ndim)
        t = reshard(t, mesh, want)
        return _guard_replicated_inputs(local_of(t), mesh, want, out_pl)
    largs, lkwargs = _map_tensors(args, conv), _map_tensors(kwargs, conv)
    with torch._C.DisableTorchFunctionSubclass():
        out = func(*largs, **lkwargs)
    return _wrap_out(out, mesh, out_pl)


def _matmul(func, args, kwargs, mesh, name):
    x, w = args[0], args[1]
    bias = args[2] if len(args) > 2 else kwargs.get("bias")
    if name == "linear":      # torch linear: weight is [out, in]
        return _fallback(func, args, kwargs, mesh)
    rep = [Replicate()] * mesh.ndim
    xp = x._dist_placements if is_dist(x) else rep
    wp = w._dist_placements if is_dist(w) else rep
    xnd = len(x.shape) if is_dist(x) else x.dim()
    wnd = len(w.shape) if is_dist(w) else w.dim()
    if wnd != 2 or xnd < 2:
        return _fallback(func, args, kwargs, mesh)
    out_pl, xw, ww = [], [], []
    for a in range(mesh.ndim):
        px, pw = xp[a], wp[a]
        if px.is_partial():
            px = Replicate()
        if pw.is_partial():
            pw = Replicate()
        if px.is_shard() and px.dim < xnd - 1 and pw.is_replicated():
            out_pl.append(Shard(px.dim)); xw.append(px); ww.append(pw)
        elif px.is_replicated() and pw.is_shard() and pw.dim == 1:
            out_pl.append(Shard(xnd - 1)); xw.append(px); ww.append(pw)
        elif px.is_shard() and px.dim == xnd - 1 and pw.is_shard() and pw.dim == 0:
            out_pl.append(Partial()); xw.append(px); ww.append(pw)
        elif px.is_replicated() and pw.is_shard() and pw.dim == 0:
            out_pl.append(Partial()); xw.append(Shard(xnd - 1)); ww.append(pw)      # slice x locally, no traffic
        else:
            out_pl.append(Replicate()); xw.append(Replicate()); ww.append(Replicate())
    x = x if is_dist(x) else DistTensor.wrap(_plain(x), mesh, rep)
    w = w if is_dist(w) else DistTensor.wrap(_plain(w), mesh, rep)
    xl = _guard_replicated_inputs(local_of(reshard(x, mesh, xw)), mesh, xw, out_pl)
    wl = _guard_replicated_inputs(local_of(reshard(w, mesh, ww)), mesh, ww, out_pl)
    out = torch.matmul(xl, wl)
    return DistTensor.wrap(out, mesh, out_pl)


def _reduce(func, args, kwargs, mesh, name):
    x = args[0]
    dims = kwargs.get("dim", kwargs.get("axis", args[1] if len(args) > 1 else None))
    keep = kwargs.get("keepdim", args[2] if len(args) > 2 else False)
    nd = len(x.shape)
    if any(p.is_partial() for p in x._dist_placements):
        return _fallback(func, args, kwargs, mesh)
    if dims is None or (isinstance(dims, (list, tuple)) and len(dims) == 0):
        rdims = list(range(nd))
    else:
        rdims = [d % nd for d in (dims if isinstance(dims, (list, tuple)) else [dims])]
    out_pl = []
    for p in x._dist_placements:
        if p.is_shard() and p.dim in rdims:
            out_pl.append(Partial(ReduceType.kRedAvg if name == "mean" else ReduceType.kRedSum))
        elif p.is_shard():
            out_pl.append(Shard(p.dim if keep else p.dim - sum(1 for d in rdims if d < p.dim)))
        else:
            out_pl.append(Replicate())
    return _wrap_out(_run_local(func, args, kwargs), mesh, out_pl)


def _dispatch(func, args, kwargs):
    name = getattr(func, "__name__", "")
    tensors = _flat_tensors((args, kwargs), [])
    dts = [t for t in tensors if is_dist(t)]
    if name in ("__get__", "__set__", "__delete__") or name in _META or not dts:
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)
    mesh = dts[0]._dist_mesh
    if any(t._dist_mesh != mesh for t in dts):
        raise ValueError("operands live on different process meshes; reshard one of them first")
    if mesh.coord_of(C.get_rank()) is None:      # this rank holds no part of the mesh: nothing to compute
        return dts[0]
    if name in ("matmul", "mm", "linear") and len(args) >= 2:
        return _matmul(func, args, kwargs, mesh, name)
    if name in _REDUCE and is_dist(args[0]):
        return _reduce(func, args, kwargs, mesh, name)
    if name in _ELEMENTWISE:
        if any(p.is_partial() for t in dts for p in t._dist_placements):
            unp = lambda t: reshard(t, mesh, [Replicate() if p.is_partial() else p for p in t._dist_placements]) \
                if is_dist(t) else t    # noqa: E731
            args, kwargs = _map_tensors(args, unp), _map_tensors(kwargs, unp)
            tensors = _flat_tensors((args, kwargs), [])
        return _elementwise(func, args, kwargs, mesh, tensors)
    if name in _ROWWISE and is_dist(args[0]):
        x = args[0]
        nd = len(x.shape)
        dim = kwargs.get("dim", args[1] if (len(args) > 1 and isinstance(args[1], int)) else -1)
        others_plain = all(not is_dist(t) or t is x or all(p.is_replicated() for p in t._dist_placements) for t in tensors)
        if others_plain and not any(p.is_partial() or (p.is_shard() and p.dim == dim % nd) for p in x._dist_placements) \
                and (name in ("softmax", "log_softmax") or not any(p.is_shard() and p.dim == nd - 1
                                                                   for p in x._dist_placements)):
            pl = x._dist_placements
            conv = lambda t: _guard_replicated_inputs(local_of(t), mesh, t._dist_placements, pl) \
                if is_dist(t) else _plain(t)    # noqa: E731
            with torch._C.DisableTorchFunctionSubclass():
                out = func(*_map_tensors(args, conv), **_map_tensors(kwargs, conv))
            return _wrap_out(out, mesh, pl)
    if name in ("transpose", "permute", "t") and is_dist(args[0]):
        x = args[0]
        nd = len(x.shape)
        if name == "t":
            perm = [1, 0] if nd == 2 else list(range(nd))
        elif name == "transpose":
            d0, d1 = args[1] % nd, args[2] % nd
            perm = list(range(nd)); perm[d0], perm[d1] = d1, d0
        else:
            perm = list(args[1]) if isinstance(args[1], (list, tuple)) else list(args[1:])
            perm = [p % nd for p in perm]
        pl = [Shard(perm.index(p.dim)) if p.is_shard() else p for p in x._dist_placements]
        return _wrap_out(_run_local(func, args, kwargs), mesh, pl)
    if name in ("reshape", "view", "flatten") and is_dist(args[0]):
        x = args[0]
        pl = x._dist_placements
        shard_dims = [p.dim for p in pl if p.is_shard()]
        if not any(p.is_partial() for p in pl) and shard_dims in ([], [0]):
            if not shard_dims:
                return _wrap_out(_run_local(func, args, kwargs), mesh, pl)
            # sharded on dim 0: valid when the target keeps dim 0 as the outermost factor
            g = x.shape
            n = [mesh.shape[a] for a, p in enumerate(pl) if p.is_shard()][0]
            if name == "flatten":
                start = kwargs.get("start_dim", args[1] if len(args) > 1 else 0)
                if start % len(g) >= 0:
                    return _wrap_out(_run_local(func, args, kwargs), mesh, pl)
            else:
                tgt = list(args[1]) if isinstance(args[1], (list, tuple, torch.Size)) else list(args[1:])
                numel = 1
                for s in g:
                    numel *= s
                if tgt.count(-1) == 1:
                    known = 1
                    for s in tgt:
                        known *= s if s != -1 else 1
                    tgt[tgt.index(-1)] = numel // known
                if tgt and tgt[0] % n == 0 and tgt[0] >= g[0] and tgt[0] % g[0] == 0 or (tgt and tgt[0] == g[0]):
                    ltgt = [tgt[0] // n] + tgt[1:]
                    with torch._C.DisableTorchFunctionSubclass():
                        out = local_of(x).reshape(ltgt)
                    return DistTensor.wrap(out, mesh, pl)
    if name == "cross_entropy" and is_dist(args[0]):
        x, lab = args[0], args[1]
        red = kwargs.get("reduction", "mean")
        pl = x._dist_placements
        ok = all(p.is_replicated() or (p.is_shard() and p.dim == 0) for p in pl) and red in ("mean", "sum", "none") \
            and kwargs.get("weight") is None and kwargs.get("ignore_index", -100) < 0 and x.dim() == 2
        if ok:
            lab_d = lab if is_dist(lab) else DistTensor.wrap(_plain(lab), mesh, [Replicate()] * mesh.ndim)
            lab_l = local_of(reshard(lab_d, mesh, pl))
            with torch._C.DisableTorchFunctionSubclass():
                out = func(local_of(x), lab_l, *args[2:], **kwargs)
            if red == "none":
                return DistTensor.wrap(out, mesh, pl)
            rt = ReduceType.kRedAvg if red == "mean" else ReduceType.kRedSum
            return DistTensor.wrap(out, mesh, [Partial(rt) if p.is_shard() else p for p in pl])
    if name == "embedding" and len(args) >= 2:
        ids, w = args[0], args[1]
        wp = w._dist_placements if is_dist(w) else [Replicate()] * mesh.ndim
        ip = ids._dist_placements if is_dist(ids) else [Replicate()] * mesh.ndim
        if all(p.is_replicated() for p in wp) and not any(p.is_partial() for p in ip):
            wl = _guard_replicated_inputs(local_of(w) if is_dist(w) else _plain(w), mesh, wp, ip)
            with torch._C.DisableTorchFunctionSubclass():
                out = func(local_of(ids) if is_dist(ids) else _plain(ids), wl, *args[2:], **kwargs)
            return DistTensor.wrap(out, mesh, ip)
    if name in ("__getitem__", "__setitem__", "__repr__", "__str__", "item", "tolist", "numpy", "__bool__", "__float__",
                "__int__", "allclose", "equal"):
        return _fallback(func, args, kwargs, mesh) if name == "__getitem__" else _run_on_full(func, args, kwargs, mesh)
    out = _rule_dispatch(name, func, args, kwargs, mesh)
    if out is not NotImplemented:
        return out
    return _fallback(func, args, kwargs, mesh)


# --------------------------------------------------------------------------- operators driven by the SPMD rule registry
def _spec_of(t, mesh):
    from .spmd_rules import DistTensorSpec
    if not is_dist(t):
        return DistTensorSpec(list(t.shape), [-1] * t.dim())
    dm = [-1] * len(t.shape)
    for a, p in enumerate(t._dist_placements):
        if p.is_shard():
            dm[p.dim] = a
    return DistTensorSpec(list(t.shape), dm)


def _placements_of(sp, mesh):
    pl = [Replicate()] * mesh.ndim
    for d, a in enumerate(sp.dims_mapping):
        if a != -1:
            pl[a] = Shard(d)
    for a in sp.partial_dims:
        pl[a] = Partial()
    return pl


def _by_rule(rule_name, tensors, attrs, mesh, call, list_input=False, rule_kwargs=None):
    """Run ``call(local tensors)`` with the inputs re-sharded as the rule ``rule_name`` asks and wrap the result(s) with the
    placements it infers.  ``tensors``: the tensor inputs in the rule's order (``None`` entries are passed through)."""
    from .spmd_rules import get_phi_spmd_rule
    rep = [Replicate()] * mesh.ndim
    dts = []
    for t in tensors:
        if t is None:
            dts.append(None)
            continue
        d = t if is_dist(t) else DistTensor.wrap(_plain(t), mesh, rep)
        if any(p.is_partial() for p in d._dist_placements):
            d = reshard(d, mesh, [Replicate() if p.is_partial() else p for p in d._dist_placements])
        dts.append(d)
    specs = [None if d is None else _spec_of(d, mesh) for d in dts]
    rule = get_phi_spmd_rule(rule_name)
    new_in, outs = rule.infer_forward(specs, *attrs, **(rule_kwargs or {})) if list_input else \
        rule.infer_forward(*specs, *attrs, **(rule_kwargs or {}))
    if list_input:
        new_in = new_in[0]
    flat_outs = outs[0] if (outs and isinstance(outs[0], list)) else outs
    ref_pl = _placements_of(flat_outs[0], mesh) if flat_outs else rep
    it = iter(new_in)
    locals_ = []
    for d in dts:
        if d is None:
            locals_.append(None)
            continue
        want = _placements_of(next(it), mesh)
        d = reshard(d, mesh, want)
        locals_.append(_guard_replicated_inputs(local_of(d), mesh, want, ref_pl))
    with torch._C.DisableTorchFunctionSubclass():
        out = call(locals_)
    if isinstance(out, (tuple, list)):
        pls = [_placements_of(o, mesh) for o in flat_outs]
        pls += [pls[-1] if pls else rep] * (len(out) - len(pls))
        return type(out)(DistTensor.wrap(o, mesh, pl) if isinstance(o, torch.Tensor) else o for o, pl in zip(out, pls))
    return DistTensor.wrap(out, mesh, ref_pl)


def _arg(args, kwargs, pos, name, default=None):
    if name in kwargs:
        return kwargs[name]
    return args[pos] if len(args) > pos else default


def _rule_dispatch(name, func, args, kwargs, mesh):
    """Operators whose sharded dims pass through untouched: the rule decides which dims must be gathered first, the local
    call then takes the same arguments as the global one.  Returns NotImplemented when the operator is not covered."""
    if name in ("cat", "concat", "concatenate", "stack") and isinstance(args[0], (list, tuple)):
        xs = list(args[0])
        dim = _arg(args, kwargs, 1, "dim", kwargs.get("axis", 0))
        kw = {k: v for k, v in kwargs.items() if k not in ("dim", "axis")}
        return _by_rule("stack" if name == "stack" else "concat", xs, (dim,), mesh, lambda ls: func(ls, dim, **kw), list_input=True)
    x = args[0] if args else None
    if not is_dist(x):
        return NotImplemented
    nd = len(x.shape)
    if name in ("split", "chunk", "tensor_split", "split_with_sizes"):
        arg = _arg(args, kwargs, 1, "split_size_or_sections", kwargs.get("chunks", kwargs.get("split_size", kwargs.get("split_sizes"))))
        dim = _arg(args, kwargs, 2, "dim", 0)
        size = x.shape[dim]
        if name == "chunk" or name == "tensor_split":
            step = -(-size // arg)
            sections = [min(step, size - i) for i in range(0, size, step)]
        else:
            sections = list(arg) if isinstance(arg, (list, tuple)) else [min(arg, size - i) for i in range(0, size, arg)]
        return _by_rule("split", [x], (sections, dim), mesh, lambda ls: tuple(torch.split(ls[0], sections, dim)))
    if name == "unbind":
        dim = _arg(args, kwargs, 1, "dim", 0)
        return _by_rule("unbind", [x], (dim,), mesh, lambda ls: tuple(torch.unbind(ls[0], dim)))
    if name == "squeeze":
        dim = _arg(args, kwargs, 1, "dim", None)
        return _by_rule("squeeze", [x], (dim if dim is None else (list(dim) if isinstance(dim, (list, tuple)) else [dim]),), mesh,
                        lambda ls: func(ls[0]) if dim is None else func(ls[0], dim))
    if name == "unsqueeze":
        dim = _arg(args, kwargs, 1, "dim")
        return _by_rule("unsqueeze", [x], ([dim],), mesh, lambda ls: func(ls[0], dim))
    if name in ("cumsum", "cumprod", "logcumsumexp"):
        dim = _arg(args, kwargs, 1, "dim", -1)
        kw = {k: v for k, v in kwargs.items() if k != "dim"}
        return _by_rule("cumsum", [x], (dim,), mesh, lambda ls: func(ls[0], dim, **kw))
    if name in ("argmax", "argmin"):
        dim = _arg(args, kwargs, 1, "dim", None)
        keep = _arg(args, kwargs, 2, "keepdim", False)
        return _by_rule("argmax", [x], (dim, keep, dim is None), mesh, lambda ls: func(ls[0], dim, keep))
    if name in ("max", "min", "amax", "amin", "prod", "all", "any", "logsumexp") and (len(args) > 1 or "dim" in kwargs) \
            and not isinstance(_arg(args, kwargs, 1, "dim"), torch.Tensor):
        dim = _arg(args, kwargs, 1, "dim")
        keep = _arg(args, kwargs, 2, "keepdim", False)
        # the local call must see the whole reduced dim: use the non-partial form of the rule
        return _by_rule("logsumexp", [x], (dim, keep), mesh, lambda ls: func(ls[0], dim, keep))
    if name == "one_hot":
        n = _arg(args, kwargs, 1, "num_classes", -1)
        if n is None or n < 0:
            return NotImplemented
        return _by_rule("one_hot", [x], (n,), mesh, lambda ls: func(ls[0], n))
    if name in ("triu", "tril"):
        diag = _arg(args, kwargs, 1, "diagonal", 0)
        return _by_rule("triu", [x], (diag,), mesh, lambda ls: func(ls[0], diag))
    if name in ("tile", "repeat"):
        reps = list(args[1]) if (len(args) > 1 and isinstance(args[1], (list, tuple, torch.Size))) else list(args[1:]) or list(kwargs.get("dims", ()))
        return _by_rule("tile", [x], (reps,), mesh, lambda ls: ls[0].repeat(*([1] * (nd - len(reps)) + reps)) if len(reps) < nd else ls[0].repeat(*reps))
    if name in ("expand", "broadcast_to", "expand_as"):
        if name == "expand_as":
            other = args[1]
            tgt = list(other.shape)
        else:
            tgt = list(args[1]) if (len(args) > 1 and isinstance(args[1], (list, tuple, torch.Size))) else list(args[1:]) or list(kwargs.get("size", ()))
        off = len(tgt) - nd
        tgt = [x.shape[i - off] if (s == -1 and i >= off) else s for i, s in enumerate(tgt)]

        def call(ls):
            loc = list(tgt)
            for i, s in enumerate(ls[0].shape):            # dims that are carried over keep their local size
                if x.shape[i] != 1 or tgt[off + i] == 1:
                    loc[off + i] = s
            return ls[0].expand(loc)
        return _by_rule("expand_as", [x], (None, tgt), mesh, call)
    if name == "pad":
        pads = list(_arg(args, kwargs, 1, "pad"))
        kw = {k: v for k, v in kwargs.items() if k != "pad"}
        rest = args[2:]
        # torch lists pads from the last dim backwards; the rule takes (before, after) per dim from dim 0
        per_dim = [0] * (2 * nd)
        for i in range(len(pads) // 2):
            d = nd - 1 - i
            per_dim[2 * d], per_dim[2 * d + 1] = pads[2 * i], pads[2 * i + 1]
        return _by_rule("pad", [x], (per_dim,), mesh, lambda ls: func(ls[0], pads, *rest, **kw))
    if name == "index_select":
        dim, index = args[1], args[2]
        return _by_rule("gather", [x, index], (dim,), mesh, lambda ls: func(ls[0], dim, ls[1]))
    if name == "scaled_dot_product_attention" and len(args) >= 3:
        q, k, v = args[:3]
        mask = _arg(args, kwargs, 3, "attn_mask", None)
        kw = {kk: vv for kk, vv in kwargs.items() if kk != "attn_mask"}
        # torch layout is [batch, heads, seq, head_dim]; the rule speaks [batch, seq, heads, head_dim]
        from .spmd_rules import DistTensorSpec, get_phi_spmd_rule
        rep = [Replicate()] * mesh.ndim
        ds = [t if is_dist(t) else DistTensor.wrap(_plain(t), mesh, rep) for t in (q, k, v)]
        ds = [reshard(d, mesh, [Replicate() if p.is_partial() else p for p in d._dist_placements]) for d in ds]
        sw = lambda sp: DistTensorSpec([sp.shape[0], sp.shape[2], sp.shape[1], sp.shape[3]],     # noqa: E731
                                       [sp.dims_mapping[0], sp.dims_mapping[2], sp.dims_mapping[1], sp.dims_mapping[3]])
        new_in, outs = get_phi_spmd_rule("flash_attention").infer_forward(*[sw(_spec_of(d, mesh)) for d in ds])
        out_pl = _placements_of(sw(outs[0]), mesh)
        ls = []
        for d, sp in zip(ds, new_in):
            want = _placements_of(sw(sp), mesh)
            ls.append(_guard_replicated_inputs(local_of(reshard(d, mesh, want)), mesh, want, out_pl))
        m_local = None
        if mask is not None:
            md = mask if is_dist(mask) else DistTensor.wrap(_plain(mask), mesh, rep)
            want = [Replicate()] * mesh.ndim
            for a, p in enumerate(out_pl):              # the mask follows the batch / head split where it has those dims
                if p.is_shard() and p.dim < 2 and len(md.shape) == 4 and md.shape[p.dim] != 1:
                    want[a] = Shard(p.dim)
            m_local = local_of(reshard(md, mesh, want))
        with torch._C.DisableTorchFunctionSubclass():
            out = func(ls[0], ls[1], ls[2], m_local, *args[4:], **kw) if mask is not None or len(args) > 3 else func(ls[0], ls[1], ls[2], **kw)
        return DistTensor.wrap(out, mesh, out_pl)
    return NotImplemented


def _run_on_full(func, args, kwargs, mesh):
    conv = lambda t: local_of(_to_replicated(t, mesh)).as_subclass(Tensor) if is_dist(t) else t   # noqa: E731
    with torch._C.DisableTorchFunctionSubclass():
        return func(*_map_tensors(args, conv), **_map_tensors(kwargs, conv))
