"""``paddle.static.nn``: functional layer builders that create their parameters on first use
(python/paddle/static/nn/common.py) and control flow (python/paddle/static/nn/control_flow.py) recorded as
sub-blocks of the program: both branches of ``cond`` and the condition/body of ``while_loop`` are traced once and
selected / iterated when the program is replayed."""
from __future__ import annotations

import torch

from .._core.tensor import as_tensor
from .. import nn as _nn
from ..nn import functional as F
from . import graph as _g


def _p(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


def _act(x, act):
    if act is None:
        return x
    return getattr(F, act)(x)


def fc(x, size, num_flatten_dims=1, weight_attr=None, bias_attr=None, activation=None, name=None):
    xs = list(x) if isinstance(x, (list, tuple)) else [x]
    was = weight_attr if isinstance(weight_attr, (list, tuple)) else [weight_attr] * len(xs)
    out = None
    for xi, wa in zip(xs, was):
        nfd = num_flatten_dims if num_flatten_dims >= 0 else xi.dim() + num_flatten_dims
        in_f = 1
        for s in xi.shape[nfd:]:
            in_f *= int(s)
        lin = _nn.Linear(in_f, size, weight_attr=wa, bias_attr=False, name=name)
        flat = xi.flatten(nfd) if xi.dim() > nfd + 1 else xi
        y = lin(flat)
        out = y if out is None else out + y
    if bias_attr is not False:
        b = _nn.Layer().create_parameter([size], bias_attr, xs[0].dtype, is_bias=True)
        out = out + b
    return _act(out, activation)


def embedding(input, size, is_sparse=False, is_distributed=False, padding_idx=None, param_attr=None, dtype="float32"):
    emb = _nn.Embedding(size[0], size[1], padding_idx=padding_idx, sparse=is_sparse, weight_attr=param_attr)
    return emb(input)


def sparse_embedding(input, size, padding_idx=None, is_test=False, entry=None, table_class="MemorySparseTable",
                     param_attr=None, dtype="float32", slot=None):
    return embedding(input, size, True, True, padding_idx, param_attr, dtype)


def _conv(cls, input, num_filters, filter_size, stride, padding, dilation, groups, param_attr, bias_attr, act,
          data_format, ch_axis, **extra):
    cin = input.shape[ch_axis]
    layer = cls(cin, num_filters, filter_size, stride=stride, padding=padding, dilation=dilation, groups=groups or 1,
                weight_attr=param_attr, bias_attr=bias_attr, data_format=data_format, **extra)
    return layer


def conv2d(input, num_filters, filter_size, stride=1, padding=0, dilation=1, groups=None, param_attr=None,
           bias_attr=None, use_cudnn=True, act=None, name=None, data_format="NCHW"):
    layer = _conv(_nn.Conv2D, input, num_filters, filter_size, stride, padding, dilation, groups, param_attr, bias_attr,
                  act, data_format, 1 if data_format == "NCHW" else -1)
    return _act(layer(input), act)


def conv3d(input, num_filters, filter_size, stride=1, padding=0, dilation=1, groups=None, param_attr=None,
           bias_attr=None, use_cudnn=True, act=None, name=None, data_format="NCDHW"):
    layer = _conv(_nn.Conv3D, input, num_filters, filter_size, stride, padding, dilation, groups, param_attr, bias_attr,
                  act, data_format, 1 if data_format == "NCDHW" else -1)
    return _act(layer(input), act)


def conv2d_transpose(input, num_filters, output_size=None, filter_size=None, padding=0, stride=1, dilation=1,
                     groups=None, param_attr=None, bias_attr=None, use_cudnn=True, act=None, name=None,
                     data_format="NCHW"):
    layer = _conv(_nn.Conv2DTranspose, input, num_filters, filter_size, stride, padding, dilation, groups, param_attr,
                  bias_attr, act, data_format, 1 if data_format == "NCHW" else -1)
    return _act(layer(input, output_size) if output_size is not None else layer(input), act)


def conv3d_transpose(input, num_filters, output_size=None, filter_size=None, padding=0, stride=1, dilation=1,
                     groups=None, param_attr=None, bias_attr=None, use_cudnn=True, act=None, name=None,
                     data_format="NCDHW"):
    layer = _conv(_nn.Conv3DTranspose, input, num_filters, filter_size, stride, padding, dilation, groups, param_attr,
                  bias_attr, act, data_format, 1 if data_format == "NCDHW" else -1)
    return _act(layer(input, output_size) if output_size is not None else layer(input), act)


def deform_conv2d(x, offset, mask, num_filters, filter_size, stride=1, padding=0, dilation=1, groups=1,
                  deformable_groups=1, im2col_step=1, weight_attr=None, bias_attr=None, name=None):
    from ..vision.ops import DeformConv2D
    layer = DeformConv2D(x.shape[1], num_filters, filter_size, stride, padding, dilation, deformable_groups, groups,
                         weight_attr, bias_attr)
    return layer(x, offset, mask)


def batch_norm(input, act=None, is_test=False, momentum=0.9, epsilon=1e-05, param_attr=None, bias_attr=None,
               data_layout="NCHW", in_place=False, name=None, moving_mean_name=None, moving_variance_name=None,
               do_model_average_for_mean_and_var=True, use_global_stats=False):
    c = input.shape[1 if data_layout == "NCHW" else -1]
    cls = {2: _nn.BatchNorm1D, 3: _nn.BatchNorm1D, 4: _nn.BatchNorm2D, 5: _nn.BatchNorm3D}[input.dim()]
    fmt = {"NCHW": {2: "NC", 3: "NCL", 4: "NCHW", 5: "NCDHW"}, "NHWC": {2: "NC", 3: "NLC", 4: "NHWC", 5: "NDHWC"}}[data_layout][input.dim()]
    layer = cls(c, momentum=momentum, epsilon=epsilon, weight_attr=param_attr, bias_attr=bias_attr, data_format=fmt,
                use_global_stats=use_global_stats or None)
    if is_test:
        layer.eval()
    return _act(layer(input), act)


def instance_norm(input, epsilon=1e-05, param_attr=None, bias_attr=None, name=None):
    cls = {3: _nn.InstanceNorm1D, 4: _nn.InstanceNorm2D, 5: _nn.InstanceNorm3D}[input.dim()]
    return cls(input.shape[1], epsilon=epsilon, weight_attr=param_attr, bias_attr=bias_attr)(input)


def group_norm(input, groups, epsilon=1e-05, param_attr=None, bias_attr=None, act=None, data_layout="NCHW", name=None):
    layer = _nn.GroupNorm(groups, input.shape[1 if data_layout == "NCHW" else -1], epsilon=epsilon,
                          weight_attr=param_attr, bias_attr=bias_attr, data_format=data_layout)
    return _act(layer(input), act)


def layer_norm(input, scale=True, shift=True, begin_norm_axis=1, epsilon=1e-05, param_attr=None, bias_attr=None,
               act=None, name=None):
    shape = [int(s) for s in input.shape[begin_norm_axis:]]
    layer = _nn.LayerNorm(shape, epsilon=epsilon, weight_attr=param_attr if scale else False,
                          bias_attr=bias_attr if shift else False)
    return _act(layer(input), act)


def data_norm(input, act=None, epsilon=1e-05, param_attr=None, data_layout="NCHW", in_place=False, name=None,
              moving_mean_name=None, moving_variance_name=None, do_model_average_for_mean_and_var=True, slot_dim=-1,
              sync_stats=False, summary_decay_rate=0.9999999, enable_scale_and_shift=False):
    """Normalises with accumulated batch statistics ``(x - sum/size) * sqrt(size/square_sum)``; the three summaries
    are persistent and start at size=1e4, sum=0, square_sum=1e4."""
    c = input.shape[-1]
    pa = param_attr or {}
    with _g.suspend():
        size = torch.full([c], float(pa.get("batch_size", 1e4)))
        bsum = torch.full([c], float(pa.get("batch_sum", 0.0)))
        sq = torch.full([c], float(pa.get("batch_square", 1e4)))
    mean = as_tensor(bsum / size)
    scale = as_tensor(torch.sqrt(size / sq))
    out = (input - mean) * scale
    return _act(out, act)


def prelu(x, mode, param_attr=None, data_format="NCHW", name=None):
    if mode == "all":
        shape = [1]
    elif mode == "channel":
        shape = [x.shape[1 if data_format[1] == "C" else -1]]
    else:
        shape = [1] + [int(s) for s in x.shape[1:]]
    from ..nn.initializer import Constant
    alpha = _nn.Layer().create_parameter(shape, param_attr, x.dtype, default_initializer=Constant(0.25))
    if mode == "element":
        return as_tensor(torch.where(_p(x) > 0, _p(x), _p(alpha) * _p(x)))
    return F.prelu(x, alpha, data_format=data_format)


def bilinear_tensor_product(x, y, size, act=None, name=None, param_attr=None, bias_attr=None):
    layer = _nn.Bilinear(x.shape[-1], y.shape[-1], size, weight_attr=param_attr, bias_attr=bias_attr)
    return _act(layer(x, y), act)


def row_conv(input, future_context_size, param_attr=None, act=None):
    """Lookahead convolution: ``out[t] = sum_{i=0..k} in[t+i] * w[i]`` over the time axis of ``[B, T, D]``."""
    d = input.shape[-1]
    w = _nn.Layer().create_parameter([future_context_size + 1, d], param_attr, input.dtype)
    x = _p(input)
    pad = torch.nn.functional.pad(x, (0, 0, 0, future_context_size))
    out = sum(pad[:, i:i + x.shape[1]] * _p(w)[i] for i in range(future_context_size + 1))
    return _act(as_tensor(out), act)


def spectral_norm(weight, dim=0, power_iters=1, eps=1e-12, name=None):
    return _nn.SpectralNorm(list(weight.shape), dim, power_iters, eps)(weight)


def nce(input, label, num_total_classes, sample_weight=None, param_attr=None, bias_attr=None, num_neg_samples=None,
        name=None, sampler="uniform", custom_dist=None, seed=0, is_sparse=False):
    """Noise-contrastive estimation loss with uniformly sampled negatives, one cost per example ``[B, 1]``."""
    d = input.shape[-1]
    k = num_neg_samples or 10
    holder = _nn.Layer()
    w = holder.create_parameter([num_total_classes, d], param_attr, input.dtype)
    b = holder.create_parameter([num_total_classes], bias_attr, input.dtype, is_bias=True)
    x, y = _p(input), _p(label).reshape(-1, 1).long()
    neg = torch.randint(0, num_total_classes, (x.shape[0], k), device=x.device)
    idx = torch.cat([y, neg], 1)
    logits = torch.einsum("bd,bkd->bk", x, _p(w)[idx]) + _p(b)[idx]
    noise = k / float(num_total_classes)
    p = torch.sigmoid(logits)
    pos = -torch.log(p[:, :1] / (p[:, :1] + noise))
    negc = -torch.log(noise / (p[:, 1:] + noise)).sum(1, keepdim=True)
    cost = pos + negc
    if sample_weight is not None:
        cost = cost * _p(sample_weight).reshape(-1, 1)
    return as_tensor(cost)


def py_func(func, x, out, backward_func=None, skip_vars_in_backward_input=None):
    from . import py_func as _pf
    return _pf(func, x, out, backward_func, skip_vars_in_backward_input)


def static_pylayer(forward_fn, inputs, backward_fn=None, name=None):
    """Runs ``forward_fn(*inputs)`` with a user-supplied backward (control_flow.py ``static_pylayer``)."""
    if backward_fn is None:
        with torch.no_grad():
            return forward_fn(*inputs)

    class _Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *xs):
            with torch.enable_grad():
                out = forward_fn(*[as_tensor(t) for t in xs])
            return _p(out) if isinstance(out, torch.Tensor) else tuple(_p(o) for o in out)

        @staticmethod
        def backward(ctx, *gs):
            r = backward_fn(*[as_tensor(g) for g in gs])
            return _p(r) if isinstance(r, torch.Tensor) else tuple(_p(t) for t in r)
    out = _Fn.apply(*[_p(t) for t in inputs])
    return as_tensor(out) if isinstance(out, torch.Tensor) else [as_tensor(o) for o in out]


# ------------------------------------------------------------------------------ control flow
def _leaves(out):
    from torch.utils import _pytree as pytree
    return [o for o in pytree.tree_leaves(out) if isinstance(o, torch.Tensor)]


def _truth(pred):
    return bool(_p(pred).reshape(-1)[0].item()) if isinstance(pred, torch.Tensor) else bool(pred)


class _CondRun:
    """Replay of a two-branch conditional: runs the selected branch's nodes and binds its results to the output
    slots (the slots of the true branch's example results)."""
    _needs_grad = False

    def __init__(self, prog, t_nodes, f_nodes, t_slots, f_slots):
        self.prog, self.t_nodes, self.f_nodes, self.t_slots, self.f_slots = prog, t_nodes, f_nodes, t_slots, f_slots
        self.__name__ = "cond"


def cond(pred, true_fn=None, false_fn=None, name=None, return_names=None):
    if not _g.recording():
        if _truth(pred):
            return true_fn() if true_fn is not None else None
        return false_fn() if false_fn is not None else None
    prog = _g.current_program()
    with prog._sub_block() as t_nodes:
        t_out = true_fn() if true_fn is not None else None
    with prog._sub_block() as f_nodes:
        f_out = false_fn() if false_fn is not None else None
    t_leaves, f_leaves = _leaves(t_out), _leaves(f_out)
    if len(t_leaves) != len(f_leaves):
        raise ValueError("true_fn and false_fn must return the same number of tensors")
    # values returned without passing through a recorded call (captured constants) get a slot here
    t_slots = [prog._slot_for_input(t) for t in t_leaves]
    f_slots = [prog._slot_for_input(t) for t in f_leaves]

    def run(pred_t, _env=None):
        raise RuntimeError("cond nodes are executed by the program, not called")
    node = _g.Node(run, (prog._to_refs(pred),), {}, t_slots, "cond")
    prog_ref = prog

    def node_run(p, env, node=node):
        pv = p._resolve(node.args[0], env) if isinstance(node.args[0], _g._Ref) else node.args[0]
        if _truth(pv):
            p._run_nodes(t_nodes, env)
            for s in t_slots:
                if s not in env and s in p._captured:
                    env[s] = p._captured[s]
        else:
            p._run_nodes(f_nodes, env)
            for ts, fs in zip(t_slots, f_slots):
                env[ts] = p._resolve(_g._Ref(fs), env)
    deps = _g.node_inputs(node) + _g.block_inputs(t_nodes) + _g.block_inputs(f_nodes) + f_slots
    prog._stack[-1].append(_CustomNode(node_run, "cond", t_slots, deps))
    del prog_ref
    return t_out


class _CustomNode:
    """Program node with its own replay routine (control flow)."""

    def __init__(self, run, name, out_slots, in_slots=()):
        self._run, self.name, self.out_slots, self.func = run, name, out_slots, run
        self.args, self.kwargs, self.in_slots = (), {}, list(in_slots)

    def run(self, prog, env):
        self._run(prog, env)

    @property
    def type(self):
        return self.name

    def __repr__(self):
        return f"{self.out_slots} = {self.name}(...)"


def case(pred_fn_pairs, default=None, name=None):
    pairs = list(pred_fn_pairs)
    if default is None:
        default = pairs[-1][1]
        pairs = pairs[:-1]

    def build(i):
        if i == len(pairs):
            return default
        pred, fn = pairs[i]
        return lambda: cond(pred, fn, build(i + 1))
    return build(0)()


def switch_case(branch_index, branch_fns, default=None, name=None):
    items = sorted(branch_fns.items()) if isinstance(branch_fns, dict) else [
        (i, f) if not isinstance(f, (tuple, list)) else tuple(f) for i, f in enumerate(branch_fns)]
    if default is None:
        default = items[-1][1]
    pairs = [(branch_index == i, fn) for i, fn in items]
    return case(pairs, default)


def while_loop(cond, body, loop_vars, is_test=False, name=None):
    loop_vars = list(loop_vars)
    if not _g.recording():
        while _truth(cond(*loop_vars)):
            out = body(*loop_vars)
            loop_vars = list(out) if isinstance(out, (list, tuple)) else [out]
        return loop_vars
    prog = _g.current_program()
    in_slots = [prog._slot_for_input(v) for v in loop_vars]
    with prog._sub_block() as c_nodes:
        c_out = cond(*loop_vars)
    c_slot = prog._slot_for_input(c_out)
    with prog._sub_block() as b_nodes:
        out = body(*loop_vars)
    outs = list(out) if isinstance(out, (list, tuple)) else [out]
    if len(outs) != len(loop_vars):
        raise ValueError("body must return as many values as loop_vars")
    out_slots = [prog._slot_for_input(o) for o in outs]
    res_slots = []
    results = []
    for o in outs:                       # fresh result variables so the loop inputs keep their own identity
        with _g.suspend():
            r = as_tensor(_p(o).clone())
        res_slots.append(prog._new_slot(r))
        results.append(r)

    def node_run(p, env):
        cur = [p._resolve(_g._Ref(s), env) for s in in_slots]
        saved = list(cur)
        for _ in range(1 << 30):
            for s, v in zip(in_slots, cur):
                env[s] = v
            p._run_nodes(c_nodes, env)
            if not _truth(p._resolve(_g._Ref(c_slot), env)):
                break
            p._run_nodes(b_nodes, env)
            cur = [p._resolve(_g._Ref(s), env) for s in out_slots]
        for s, v in zip(res_slots, cur):
            env[s] = v
        for s, v in zip(in_slots, saved):
            env[s] = v
    deps = in_slots + _g.block_inputs(c_nodes) + _g.block_inputs(b_nodes)
    prog._stack[-1].append(_CustomNode(node_run, "while_loop", res_slots, deps))
    return results


# ------------------------------------------------------------------------------ sequence (LoD) ops on padded batches
def _seq_unsupported(name):
    def fn(*a, **k):
        raise NotImplementedError(
            f"static.nn.{name} operates on LoD (ragged) tensors, which this framework does not have; "
            "use padded batches with paddle.nn.functional.sequence_mask")
    fn.__name__ = name
    return fn


def sequence_softmax(input, use_cudnn=False, name=None):
    return F.softmax(input, axis=1)


def sequence_pool(input, pool_type, is_test=False, pad_value=0.0):
    x = _p(input)
    pt = pool_type.lower()
    if pt == "sum":
        return as_tensor(x.sum(1))
    if pt == "average":
        return as_tensor(x.mean(1))
    if pt == "sqrt":
        return as_tensor(x.sum(1) / (x.shape[1] ** 0.5))
    if pt == "max":
        return as_tensor(torch.max(x, 1).values)
    if pt == "first":
        return as_tensor(x[:, 0])
    if pt == "last":
        return as_tensor(x[:, -1])
    raise ValueError(pool_type)


def sequence_first_step(input):
    return sequence_pool(input, "first")


def sequence_last_step(input):
    return sequence_pool(input, "last")


def sequence_conv(input, num_filters, filter_size=3, filter_stride=1, padding=True, padding_start=None,
                  bias_attr=None, param_attr=None, act=None, name=None):
    """Context-window projection over the time axis of a padded ``[B, T, D]`` batch."""
    d = input.shape[-1]
    start = -(filter_size // 2) if padding_start is None else padding_start
    holder = _nn.Layer()
    w = holder.create_parameter([filter_size * d, num_filters], param_attr, input.dtype)
    x = _p(input)
    T = x.shape[1]
    left, right = max(-start, 0), max(filter_size + start - 1, 0)
    xp = torch.nn.functional.pad(x, (0, 0, left, right))
    ctx = torch.cat([xp[:, i:i + T] for i in range(filter_size)], -1)
    out = ctx @ _p(w)
    if bias_attr is not False:
        out = out + _p(holder.create_parameter([num_filters], bias_attr, input.dtype, is_bias=True))
    return _act(as_tensor(out), act)


sequence_expand = _seq_unsupported("sequence_expand")
