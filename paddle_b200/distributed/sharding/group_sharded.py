"""``paddle.distributed.sharding.group_sharded_parallel`` - ZeRO stages 1/2/3 over one process group
(python/paddle/distributed/sharding/group_sharded.py:50; implementation classes in
fleet/meta_parallel/sharding/group_sharded_{optimizer_stage2,stage2,stage3}.py).

* ``level="os"``     optimizer state sharded: every rank updates only the parameters it owns, then owners
                     broadcast (stage 1).
* ``level="os_g"``   + gradients: each gradient is reduced to its owner as soon as it is produced and dropped
                     everywhere else (stage 2).
* ``level="p_g_os"`` + parameters: each rank stores a 1/n slice of every parameter.  A layer's parameters are
                     all-gathered into their full storage right before its forward, released right after,
                     gathered again when its backward starts, and the full gradients are reduce-scattered into
                     the slice gradients when its backward ends (stage 3; forward described in
                     group_sharded_stage3.py ``_register_forward_hooks``).  Releasing keeps the tensor object and
                     shrinks its storage to zero bytes, so tensors saved for backward stay valid once the storage
                     is filled again.
"""
from __future__ import annotations

import os

import torch

from ..._core.tensor import EagerParamBase, as_tensor
from ...nn.layer.layers import Layer
from .. import collective as C


def _numel(p):
    return int(torch.Tensor.numel(p))


def _grad_of(p):
    mg = getattr(p, "main_grad", None)
    return mg if mg is not None else torch.Tensor.grad.__get__(p)


class GroupShardedOptimizerStage2:
    """Owns the partition param -> rank (greedy by size, group_sharded_optimizer_stage2.py:283 ``_segment_params``)
    and restricts the wrapped optimizer to the local partition."""

    def __init__(self, params, optim, group=None, offload=False, dp_group=None, **kw):
        self._optim = optim
        self._group = group or C._get_default_group()
        self._rank = self._group.get_group_rank(C.get_rank())
        self._nranks = self._group.nranks
        self._all_params = list(params)
        self.offload = offload
        sizes = [0] * self._nranks
        self.param2rank, self.rank2params = {}, {r: [] for r in range(self._nranks)}
        for p in self._all_params:
            r = sizes.index(min(sizes))
            self.rank2params[r].append(p)
            self.param2rank[p.name] = r
            sizes[r] += _numel(p)
        self._local = self.rank2params[self._rank]
        local_names = {p.name for p in self._local}
        optim._param_groups = [{**g, "params": [p for p in g["params"] if p.name in local_names]}
                               for g in optim._param_groups]
        optim._parameter_list = [p for g in optim._param_groups for p in g["params"]]
        self._patch_clip()

    def _patch_clip(self):
        """Global-norm clipping needs the norm over ALL partitions: sum the local squared norms over the group."""
        from ...nn.clip import ClipGradByGlobalNorm
        clip = self._optim._grad_clip
        if isinstance(clip, ClipGradByGlobalNorm):
            inner = self._optim._global_norm_sq
            group = self._group

            def global_norm_sq(clip_, params_grads):
                sq = inner(clip_, params_grads)
                C.all_reduce(sq, group=group)
                return sq
            self._optim._global_norm_sq = global_norm_sq

    def step(self):
        self._optim.step()
        self._broadcast_params()

    def _broadcast_params(self):
        with torch.no_grad():
            for r, ps in self.rank2params.items():
                for p in ps:
                    C.broadcast(p.data, self._group.ranks[r], self._group)

    def clear_grad(self, set_to_zero=True):
        for p in self._all_params:
            g = torch.Tensor.grad.__get__(p)
            if g is not None:
                if set_to_zero:
                    g.zero_()
                else:
                    p.grad = None
            if getattr(p, "main_grad", None) is not None:
                p.main_grad.zero_()

    clear_gradients = clear_grad

    def state_dict(self):
        return self._optim.state_dict()

    def set_state_dict(self, sd):
        return self._optim.set_state_dict(sd)

    def __getattr__(self, item):
        return getattr(self._optim, item)


class GroupShardedStage2(Layer):
    """Model wrapper of stage 2: a hook on every parameter reduces its finished gradient to the owner rank
    (averaged over the group) and frees it on the other ranks (group_sharded_stage2.py ``_get_reduce_fn``)."""

    def __init__(self, layer, sharding_optimizer, group=None, sync_buffers=False, buffer_max_size=2 ** 23,
                 auto_refresh_trainable=True, device="gpu", dp_group=None, reduce_grads=True):
        super().__init__()
        self._layer = layer
        self._opt = sharding_optimizer if not isinstance(sharding_optimizer, (list, tuple)) else sharding_optimizer[0]
        self._group = group or C._get_default_group()
        self._reduce_grads = reduce_grads
        self._pending = []
        if sync_buffers:
            for b in layer.buffers():
                C.broadcast(b, self._group.ranks[0], self._group)
        for p in layer.parameters():
            C.broadcast(p.data, self._group.ranks[0], self._group)
            if p.requires_grad:
                p.register_post_accumulate_grad_hook(self._make_hook(p))
        inner_step = self._opt.step

        def step():
            self._finish_reduce()
            inner_step()
        self._opt.step = step
        # GradScaler.unscale_ runs before step(): the reductions in flight must have landed (and been averaged)
        # before gradients are unscaled and checked for inf
        self._opt._before_unscale = self._finish_reduce

    def _make_hook(self, p):
        owner = self._opt.param2rank[p.name]
        dst = self._group.ranks[owner]
        mine = owner == self._opt._rank

        def hook(param):
            g = _grad_of(param)
            if g is None:
                return
            task = C.reduce(g, dst=dst, op=C.ReduceOp.SUM, group=self._group, sync_op=False) \
                if self._reduce_grads else None
            self._pending.append((param, task, mine))
        return hook

    def _finish_reduce(self):
        n = self._group.nranks
        for param, task, mine in self._pending:
            if task is not None:
                task.wait()
            if mine:
                _grad_of(param).div_(n)
            elif self._reduce_grads:
                param.grad = None
        self._pending.clear()

    def forward(self, *a, **k):
        return self._layer(*a, **k)

    def state_dict(self, *a, **k):
        return self._layer.state_dict(*a, **k)

    def set_state_dict(self, *a, **k):
        return self._layer.set_state_dict(*a, **k)

    def parameters(self, include_sublayers=True):
        return self._layer.parameters(include_sublayers)

    def named_parameters(self, prefix="", include_sublayers=True):
        return self._layer.named_parameters(prefix, include_sublayers)


class _PreBackward(torch.autograd.Function):
    """Identity on a layer's outputs; its backward runs BEFORE the layer's own backward -> gather."""

    @staticmethod
    def forward(ctx, owner, unit, *xs):
        ctx.owner, ctx.unit = owner, unit
        return xs if len(xs) > 1 else xs[0]

    @staticmethod
    def backward(ctx, *gs):
        ctx.owner._gather(ctx.unit)
        return (None, None, *gs)


class _PostBackward(torch.autograd.Function):
    """Identity on a layer's inputs; its backward runs AFTER the layer's own backward -> reduce-scatter, release."""

    @staticmethod
    def forward(ctx, owner, unit, *xs):
        ctx.owner, ctx.unit = owner, unit
        return xs if len(xs) > 1 else xs[0]

    @staticmethod
    def backward(ctx, *gs):
        ctx.owner._reduce_and_release(ctx.unit)
        return (None, None, *gs)


class _Unit:
    """One sublayer's directly-held parameters and their slices."""

    def __init__(self, layer, params):
        self.layer, self.params = layer, params
        self.gathered = True


class GroupShardedStage3(Layer):
    def __init__(self, layer, optimizer, group=None, sync_buffers=False, device="gpu", segment_size=2 ** 20,
                 pertrain_sync_models=True, offload=False, sync_comm=False, dp_group=None, exclude_layer=None):
        super().__init__()
        self._layer = layer
        self._optim = optimizer
        self._group = group or C._get_default_group()
        self._n = self._group.nranks
        self._rank = self._group.get_group_rank(C.get_rank())
        self._exclude = set(exclude_layer or [])
        self._units = []
        self._slices = {}          # param.name -> slice parameter handed to the optimizer
        if pertrain_sync_models:
            for p in layer.parameters():
                C.broadcast(p.data, self._group.ranks[0], self._group)
        if sync_buffers:
            for b in layer.buffers():
                C.broadcast(b, self._group.ranks[0], self._group)
        self._shard_all()
        self._redirect_optimizer()
        self._register_hooks()

    # ------------------------------------------------------------------ partition
    def _padded(self, p):
        n = _numel(p)
        return (n + self._n - 1) // self._n * self._n

    def _shard_all(self):
        seen = set()
        for sub in self._layer.sublayers(include_self=True):
            if type(sub).__name__ in self._exclude or id(sub) in self._exclude:
                continue
            direct = [p for p in sub._parameters.values() if p is not None and p.requires_grad and id(p) not in seen]
            if not direct:
                continue
            for p in direct:
                seen.add(id(p))
                per = self._padded(p) // self._n
                flat = torch.zeros(self._padded(p), dtype=p.dtype, device=p.device)
                flat[:_numel(p)] = p.detach().reshape(-1)
                sl = EagerParamBase(flat[self._rank * per:(self._rank + 1) * per].clone())
                sl.name = p.name
                sl.stop_gradient = False
                p._full_shape = tuple(p.shape)
                p._full_nbytes = p.untyped_storage().nbytes()
                self._slices[p.name] = sl
            u = _Unit(sub, direct)
            self._units.append(u)
            self._release(u)
            self._try_fuse_linear(u)

    def _try_fuse_linear(self, u):
        """A Linear layer whose weight slices are whole rows runs on the fused kernels: the parameter all-gather happens
        inside the forward GEMM and again inside the input-gradient GEMM, the weight gradient is reduce-scattered by the
        GEMM that produces it (``parallel/zero3_linear.py``), and the gradient lands directly on the slice parameter.
        The full weight is then never materialised in training."""
        from ...nn.layer.common import Linear
        from ...ops import functional as K
        sub = u.layer
        u.fused_weight = None
        if type(sub) is not Linear or self._n < 2:
            return
        w = sub.weight
        if w is None or id(w) not in {id(p) for p in u.params} or len(w._full_shape) != 2:
            return
        fin, fout = w._full_shape
        if fin % self._n or w.dtype != torch.bfloat16 or not w.is_cuda or K.get_kernel_policy() != "fused":
            return
        from ...parallel import zero3_linear as Z
        sl = self._slices[w.name]
        shard = sl.view(fin // self._n, fout) if hasattr(sl, "view") else None
        if shard is None or not Z.fused_ok(C._plain(shard), self._group):
            return
        u.fused_weight = w
        owner, group, inv_n = self, self._group, 1.0 / self._n

        def forward(x, _sub=sub, _w=w):
            if _w.untyped_storage().nbytes() > 0:       # the full weight was materialised (get_all_parameters)
                from ...nn import functional as F
                return F.linear(x, _w, _sub.bias)
            sl_ = owner._slices[_w.name]
            y = Z.zero3_linear(C._plain(x), C._plain(sl_).view(fin // owner._n, fout), group, inv_n)
            if _sub.bias is not None:
                y = y + _sub.bias
            return as_tensor(y)
        sub.forward = forward

    def _redirect_optimizer(self):
        opt = self._optim
        table = self._slices
        for g in opt._param_groups:
            g["params"] = [table.get(p.name, p) for p in g["params"]]
        opt._parameter_list = [p for g in opt._param_groups for p in g["params"]]
        from ...nn.clip import ClipGradByGlobalNorm
        if isinstance(opt._grad_clip, ClipGradByGlobalNorm):
            inner, group = opt._global_norm_sq, self._group

            def global_norm_sq(clip_, params_grads):
                sq = inner(clip_, params_grads)
                C.all_reduce(sq, group=group)
                return sq
            opt._global_norm_sq = global_norm_sq

    # ------------------------------------------------------------------ gather / release
    @torch.no_grad()
    def _gather(self, u, everything=False):
        if u.gathered and not everything:
            return
        for p in u.params:
            if p is getattr(u, "fused_weight", None) and not everything:
                continue                      # gathered inside the GEMM kernels
            sl = self._slices[p.name]
            full = torch.empty(self._padded(p), dtype=p.dtype, device=sl.device)
            C.all_gather_into_tensor(full, sl.data, group=self._group)
            p.data.untyped_storage().resize_(p._full_nbytes)
            p.data.copy_(full[:_numel(p)].view(p._full_shape))
        u.gathered = True

    @torch.no_grad()
    def _release(self, u):
        for p in u.params:
            p.data.untyped_storage().resize_(0)
        u.gathered = False

    @torch.no_grad()
    def _reduce_and_release(self, u):
        for p in u.params:
            g = _grad_of(p)
            if g is None:
                continue
            sl = self._slices[p.name]
            per = self._padded(p) // self._n
            flat = torch.zeros(self._padded(p), dtype=g.dtype, device=g.device)
            flat[:_numel(p)] = g.reshape(-1)
            out = torch.empty(per, dtype=g.dtype, device=g.device)
            C.reduce_scatter(out, list(flat.chunk(self._n)), op=C.ReduceOp.SUM, group=self._group)
            out.div_(self._n)
            cur = torch.Tensor.grad.__get__(sl)
            if cur is None:
                sl.grad = out.to(sl.dtype)
            else:
                cur.add_(out.to(sl.dtype))
            p.grad = None
            if getattr(p, "main_grad", None) is not None:
                p.main_grad = None
        self._release(u)

    def _register_hooks(self):
        for u in self._units:
            def pre(layer, inputs, u=u):
                self._gather(u)
                if not torch.is_grad_enabled():
                    return None
                tens = [i for i in inputs if isinstance(i, torch.Tensor) and i.requires_grad]
                if not tens:
                    # no differentiable input (first layer): the release is driven by the outputs' hook alone
                    u._needs_tail = True
                    return None
                u._needs_tail = False
                outs = _PostBackward.apply(self, u, *tens)
                outs = outs if isinstance(outs, tuple) else (outs,)
                it = iter(outs)
                return tuple(as_tensor(next(it)) if (isinstance(i, torch.Tensor) and i.requires_grad) else i
                             for i in inputs)

            def post(layer, inputs, out, u=u):
                if torch.is_grad_enabled():
                    flat = [out] if isinstance(out, torch.Tensor) else [o for o in out if isinstance(o, torch.Tensor)]
                    flat = [o for o in flat if o.requires_grad]
                    if flat:
                        res = _PreBackward.apply(self, u, *flat)
                        res = res if isinstance(res, tuple) else (res,)
                        it = iter(res)
                        if isinstance(out, torch.Tensor):
                            out = as_tensor(next(it))
                        else:
                            out = type(out)(as_tensor(next(it)) if (isinstance(o, torch.Tensor) and o.requires_grad)
                                            else o for o in out)
                        if getattr(u, "_needs_tail", False):
                            self._tail_units.append(u)
                self._release(u)
                return out
            u.layer.register_forward_pre_hook(pre)
            u.layer.register_forward_post_hook(post)
        self._tail_units = []

    # ------------------------------------------------------------------ public surface
    def forward(self, *a, **k):
        self._tail_units = []
        return self._layer(*a, **k)

    def _finish_backward(self):
        """Units whose inputs carry no gradient (embeddings) have no post-backward node: finish them here."""
        for u in self._tail_units:
            if u.gathered:
                self._reduce_and_release(u)
        self._tail_units = []
        for u in self._units:            # anything still holding full gradients (layers called functionally)
            if any(_grad_of(p) is not None for p in u.params):
                self._reduce_and_release(u)

    @torch.no_grad()
    def get_all_parameters(self, convert2cpu=False):
        """Materialise every full parameter (for saving or evaluation outside the wrapper)."""
        for u in self._units:
            self._gather(u, everything=True)
            if convert2cpu:
                for p in u.params:
                    p.data = p.data.cpu()
        return self._layer.parameters()

    def state_dict(self, *a, **k):
        self.get_all_parameters()
        sd = {key: as_tensor(v.detach().clone()) for key, v in self._layer.state_dict(*a, **k).items()}
        for u in self._units:
            self._release(u)
        return sd

    def set_state_dict(self, sd, *a, **k):
        self.get_all_parameters()
        r = self._layer.set_state_dict(sd, *a, **k)
        with torch.no_grad():
            for u in self._units:
                for p in u.params:
                    per = self._padded(p) // self._n
                    flat = torch.zeros(self._padded(p), dtype=p.dtype, device=p.device)
                    flat[:_numel(p)] = p.detach().reshape(-1)
                    self._slices[p.name].data.copy_(flat[self._rank * per:(self._rank + 1) * per])
                self._release(u)
        return r

    def parameters(self, include_sublayers=True):
        return self._layer.parameters(include_sublayers)


class _Stage3Optimizer:
    """Optimizer facade for stage 3: finishes outstanding gradient reductions, then steps on the slices."""

    def __init__(self, optim, model):
        self._optim, self._model = optim, model

    def _before_unscale(self):
        """Called by ``GradScaler.unscale_``: the reduce-scatter of the units whose backward ran last (embeddings,
        first layer) has to finish before the gradients are unscaled, or those would be applied still multiplied
        by the loss scale."""
        self._model._finish_backward()

    def step(self):
        self._model._finish_backward()
        self._optim.step()

    def clear_grad(self, set_to_zero=True):
        for sl in self._model._slices.values():
            sl.grad = None
        self._optim.clear_grad(set_to_zero)

    clear_gradients = clear_grad

    def __getattr__(self, item):
        return getattr(self._optim, item)


class GroupShardedScaler:
    """GradScaler whose found-inf flag is agreed across the sharding group: every rank checks only the gradient
    partition it holds, so a rank that saw no inf must still skip the step when another did
    (python/paddle/distributed/fleet/meta_parallel/sharding/group_sharded_utils.py:262-330, which all-reduces the flag
    with MAX after ``check_finite_and_unscale``).  The scaler object itself is returned, with its
    ``_sync_found_inf`` hook replaced; ``GradScaler.unscale_`` calls the hook on every rank, also on one that
    holds no gradients."""

    def __new__(cls, scaler, group=None):
        g = group or C._get_default_group()

        def sync(found):
            if g is not None and g.nranks > 1:
                t = found.to(torch.int32)
                C.all_reduce(t, op=C.ReduceOp.MAX, group=g)
                found = t
            return found
        scaler._sync_found_inf = sync
        scaler._sharding_group = g
        return scaler


def group_sharded_parallel(model, optimizer, level, scaler=None, group=None, offload=False, sync_buffers=False,
                           buffer_max_size=2 ** 23, segment_size=2 ** 20, sync_comm=False, dp_group=None,
                           exclude_layer=None):
    assert level in ("os", "os_g", "p_g_os"), "level must be one of 'os', 'os_g', 'p_g_os'"
    group = group or C._get_default_group()
    if level in ("os", "os_g"):
        optimizer = GroupShardedOptimizerStage2(model.parameters(), optimizer, group=group, offload=offload,
                                                dp_group=dp_group)
        model = GroupShardedStage2(model, optimizer, group=group, sync_buffers=sync_buffers,
                                   buffer_max_size=buffer_max_size, dp_group=dp_group,
                                   reduce_grads=True)
        model._free_non_owner = level == "os_g"
    else:
        model = GroupShardedStage3(model, optimizer, group=group, sync_buffers=sync_buffers, segment_size=segment_size,
                                   offload=offload, sync_comm=sync_comm, dp_group=dp_group, exclude_layer=exclude_layer)
        optimizer = _Stage3Optimizer(optimizer, model)
    if scaler is not None:
        scaler = GroupShardedScaler(scaler, group)
    return model, optimizer, scaler


def save_group_sharded_model(model, output, optimizer=None):
    """Rank-local files ``model.pdmodel`` / ``model.pdopt`` under ``output`` (group_sharded.py:214): full
    parameters (gathered for stage 3) and this rank's optimizer partition."""
    from ...framework.io import save
    assert not os.path.isfile(output), f"Saving directory ({output}) should be a directory, not a file"
    os.makedirs(output, exist_ok=True)
    save(model.state_dict(), os.path.join(output, "model.pdmodel"))
    if optimizer is not None:
        save(optimizer.state_dict(), os.path.join(output, "model.pdopt"))
