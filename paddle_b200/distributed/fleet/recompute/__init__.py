"""Activation recompute (python/paddle/distributed/fleet/recompute/recompute.py:128 reentrant PyLayer with
RNG / AMP state replay, :463 ``recompute``, :630 ``recompute_sequential``; recompute_hybrid.py:84 partitions
saved activations over the mp group and all-gathers them on use)."""
from __future__ import annotations

import torch

from ...._core.tensor import as_tensor
from ....amp import _state as _amp_state
from ..layers.mpu.random import get_rng_state_tracker


def _rng_snapshot():
    cuda = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
    return torch.get_rng_state(), cuda, get_rng_state_tracker().get_states_tracker()


def _rng_restore(snap):
    cpu, cuda, tracker = snap
    torch.set_rng_state(cpu)
    if cuda is not None:
        torch.cuda.set_rng_state(cuda)
    get_rng_state_tracker().set_states_tracker(tracker)


class RecomputeFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_function, preserve_rng_state, offload, partition_group, n_kw, *args):
        ctx.run_function = run_function
        ctx.preserve = preserve_rng_state
        ctx.amp = dict(_amp_state)
        if preserve_rng_state:
            ctx.rng = _rng_snapshot()
        ctx.n_kw = n_kw
        ctx.tensor_idx, ctx.others = [], {}
        saved = []
        ctx.partition_group = partition_group
        ctx.offload = offload
        ctx.shapes = {}
        for i, a in enumerate(args):
            if isinstance(a, torch.Tensor):
                ctx.tensor_idx.append(i)
                t = a.detach()
                if partition_group is not None and partition_group.nranks > 1 and t.numel() % partition_group.nranks == 0:
                    ctx.shapes[i] = t.shape
                    n, r = partition_group.nranks, partition_group.rank
                    t = t.reshape(-1).chunk(n)[r].clone()
                if offload:
                    t = t.to("cpu", non_blocking=True)
                saved.append(t)
                ctx.others[i] = a.requires_grad
            else:
                ctx.others[i] = a
        ctx.save_for_backward(*saved)
        with torch.no_grad():
            out = run_function(*args)
        return out

    @staticmethod
    def backward(ctx, *grads):
        from ... import collective as C
        saved = list(ctx.saved_tensors)
        args = []
        it = iter(saved)
        n_args = len(ctx.others)
        dev = grads[0].device if grads and grads[0] is not None else None
        for i in range(n_args):
            if i in ctx.tensor_idx:
                t = next(it)
                if ctx.offload and dev is not None:
                    t = t.to(dev, non_blocking=True)
                if i in ctx.shapes:
                    parts = []
                    C.all_gather(parts, t, ctx.partition_group)
                    t = torch.cat([p.reshape(-1) for p in parts]).view(ctx.shapes[i])
                t = as_tensor(t.detach())
                t.requires_grad_(ctx.others[i])
                args.append(t)
            else:
                args.append(ctx.others[i])
        cur = _rng_snapshot() if ctx.preserve else None
        if ctx.preserve:
            _rng_restore(ctx.rng)
        prev_amp = dict(_amp_state)
        _amp_state.clear()
        _amp_state.update(ctx.amp)
        try:
            with torch.enable_grad():
                out = ctx.run_function(*args)
        finally:
            _amp_state.clear()
            _amp_state.update(prev_amp)
            if ctx.preserve:
                _rng_restore(cur)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        res = [None] * 5
        for i in range(n_args):
            a = args[i]
            res.append(a.grad if isinstance(a, torch.Tensor) and a.requires_grad else None)
        return tuple(res)


def recompute(function, *args, **kwargs):
    """Run ``function`` without storing its activations; they are recomputed during backward."""
    preserve = kwargs.pop("preserve_rng_state", True)
    use_reentrant = kwargs.pop("use_reentrant", True)
    offload = kwargs.pop("offload", False)
    group = kwargs.pop("_partition_group", None)
    if not use_reentrant:
        import torch.utils.checkpoint as cp
        return cp.checkpoint(function, *args, use_reentrant=False, preserve_rng_state=preserve, **kwargs)
    if kwargs:
        keys = list(kwargs)
        fn = function

        def function(*a):  # noqa: F811
            n = len(a) - len(keys)
            return fn(*a[:n], **dict(zip(keys, a[n:])))
        args = (*args, *[kwargs[k] for k in keys])
    out = RecomputeFunction.apply(function, preserve, offload, group, 0, *args)
    if isinstance(out, torch.Tensor):
        return as_tensor(out)
    return type(out)(as_tensor(o) if isinstance(o, torch.Tensor) else o for o in out)


def recompute_sequential(ctx, functions, *args, **kwargs):
    segments = ctx.get("segments", 1)
    preserve = ctx.get("preserve_rng_state", True)
    layers = list(functions.children()) if hasattr(functions, "children") else list(functions)
    per = max(len(layers) // segments, 1)

    def run(lo, hi):
        def f(*xs):
            x = xs[0] if len(xs) == 1 else xs
            for l in layers[lo:hi]:
                x = l(x)
            return x
        return f
    x = args
    i = 0
    while i < len(layers):
        hi = min(i + per, len(layers))
        if hi == len(layers):
            x = run(i, hi)(*(x if isinstance(x, tuple) else (x,)))
        else:
            x = recompute(run(i, hi), *(x if isinstance(x, tuple) else (x,)), preserve_rng_state=preserve)
        i = hi
    return x


# the module of the same name is imported first and the name is then re-bound to the function, as in the reference
# package (python/paddle/distributed/fleet/recompute/__init__.py)
from . import recompute as _recompute_module  # noqa: E402,F401
from .recompute_hybrid import recompute_hybrid  # noqa: E402,F401
