"""Megatron-style sequence parallelism on the model-parallel group
(python/paddle/distributed/fleet/utils/sequence_parallel_utils.py): activations between tensor-parallel
blocks are sharded along the token axis (axis 0 of ``[tokens, hidden]``).

``ColumnSequenceParallelLinear`` = all-gather then GEMM (:429), ``RowSequenceParallelLinear`` = GEMM then
reduce-scatter (:564).  With the kernel policy ``"fused"`` on CUDA bf16 both run as ONE kernel launch that
overlaps the transfer over NVLink peer memory with the tensor-core tiles
(``paddle_b200.parallel.fused_linear``); with ``"baseline"`` (or on CPU) they issue the separate,
synchronous collectives exactly where the reference does (:58-82,543-549,669-678).
"""
from __future__ import annotations

import torch

from ...._core.tensor import as_tensor
from ....nn import functional as F
from ....nn.layer.layers import Layer
from ... import collective as C
from ..layers.mpu import mp_ops
from ..layers.mpu.mp_layers import _hcg, _mark
from ..layers.mpu.random import get_rng_state_tracker


def _group(group=None):
    return group if group is not None else _hcg().get_model_parallel_group()


# ------------------------------------------------------------------ raw collectives on axis 0
def scatter(input, group=None):
    g = _group(group)
    n, r = g.nranks, g.rank
    assert input.shape[0] % n == 0, f"token count {input.shape[0]} is not divisible by the mp degree {n}"
    per = input.shape[0] // n
    return input[r * per:(r + 1) * per].contiguous()


def all_gather(input, group=None):
    g = _group(group)
    out = torch.empty((input.shape[0] * g.nranks, *input.shape[1:]), dtype=input.dtype, device=input.device)
    C.all_gather(out, input.contiguous(), g)
    return as_tensor(out)


def reduce_scatter(input, group=None):
    g = _group(group)
    assert input.shape[0] % g.nranks == 0
    out = torch.empty((input.shape[0] // g.nranks, *input.shape[1:]), dtype=input.dtype, device=input.device)
    C.reduce_scatter(out, input.contiguous(), group=g)
    return as_tensor(out)


class ScatterOp(torch.autograd.Function):
    """split along tokens (fwd) / all-gather (bwd)"""

    @staticmethod
    def forward(ctx, input, group=None):
        ctx.group = group
        return scatter(input, group)

    @staticmethod
    def backward(ctx, grad):
        return all_gather(grad, ctx.group), None


class GatherOp(torch.autograd.Function):
    """all-gather (fwd) / split (bwd)"""

    @staticmethod
    def forward(ctx, input, group=None):
        ctx.group = group
        return all_gather(input, group)

    @staticmethod
    def backward(ctx, grad):
        return scatter(grad, ctx.group), None


class AllGatherOp(torch.autograd.Function):
    """all-gather (fwd) / reduce-scatter (bwd)"""

    @staticmethod
    def forward(ctx, input, group=None):
        ctx.group = group
        return all_gather(input, group)

    @staticmethod
    def backward(ctx, grad):
        return reduce_scatter(grad, ctx.group), None


class ReduceScatterOp(torch.autograd.Function):
    """reduce-scatter (fwd) / all-gather (bwd)"""

    @staticmethod
    def forward(ctx, input, group=None):
        ctx.group = group
        return reduce_scatter(input, group)

    @staticmethod
    def backward(ctx, grad):
        return all_gather(grad, ctx.group), None


# ------------------------------------------------------------------ parameter marking + grad sync hooks
def mark_as_sequence_parallel_parameter(parameter):
    parameter.sequence_parallel = True


def is_sequence_parallel_parameter(parameter):
    return getattr(parameter, "sequence_parallel", False)


def register_sequence_parallel_allreduce_hooks(model, accumulation_steps=1, fuse_sequence_parallel_allreduce=False):
    """Norm weights / biases inside the sequence-parallel region see only their token shard, so their
    gradients are summed over the mp group every ``accumulation_steps`` backward passes (:148-216)."""
    if accumulation_steps <= 0 or not C.is_initialized():
        return
    g = _group()
    if g is None or g.nranks == 1:
        return
    params = [p for p in model.parameters() if is_sequence_parallel_parameter(p) and p.requires_grad]
    if not params:
        return
    state = {"count": 0, "total": len(params) * accumulation_steps, "per_param": {}}

    def grad_of(p):
        mg = getattr(p, "main_grad", None)
        return mg if mg is not None else torch.Tensor.grad.__get__(p)

    def reduce_all():
        grads = [gr for gr in (grad_of(p) for p in params) if gr is not None]
        by_dtype = {}
        for gr in grads:
            by_dtype.setdefault(gr.dtype, []).append(gr)
        for gs in by_dtype.values():
            flat = torch.cat([x.reshape(-1) for x in gs])
            C.all_reduce(flat, group=g)
            off = 0
            for x in gs:
                x.copy_(flat[off:off + x.numel()].view_as(x))
                off += x.numel()

    def hook(p):
        if getattr(p, "main_grad", None) is not None and torch.Tensor.grad.__get__(p) is not None:
            # main_grad was attached after this hook was registered (a sharding optimizer builds its flat gradient
            # buffers late), so this hook runs before the one that folds .grad into main_grad: fold now, the later
            # call finds nothing left to fold
            from .mix_precision_utils import _fold_grad_hook
            _fold_grad_hook(p)
        if fuse_sequence_parallel_allreduce:
            # one all-reduce of all of them, when the last one has arrived (:166-216)
            state["count"] += 1
            if state["count"] == state["total"]:
                state["count"] = 0
                reduce_all()
            return
        # per parameter, the moment its gradient is complete (:148-164): a consumer that runs from a later hook of the
        # same parameter - the sharding optimizer's bucket accounting starts a bucket's reduce-scatter under backward -
        # then sees the summed gradient
        c = state["per_param"].get(id(p), 0) + 1
        if c == accumulation_steps:
            state["per_param"][id(p)] = 0
            gr = grad_of(p)
            if gr is not None:
                C.all_reduce(gr, group=g)
        else:
            state["per_param"][id(p)] = c

    for p in params:
        if getattr(p, "main_grad", None) is not None:
            prev = getattr(p, "_main_grad_ready_hook", None)
            p._main_grad_ready_hook = (lambda prev_: (lambda q: (prev_(q) if prev_ else None, hook(q))))(prev)
        else:
            p.register_post_accumulate_grad_hook(hook)


# ------------------------------------------------------------------ layers
def _use_fused(x, weight, group, tokens_per_rank):
    from ....ops import functional as K
    from ....parallel import fused_linear
    return (x.is_cuda and x.dtype == torch.bfloat16 and K.get_kernel_policy() == "fused"
            and tokens_per_rank % 128 == 0 and fused_linear.available(x, weight, group))


class ColumnSequenceParallelLinear(Layer):
    """x: ``[tokens/n, in]`` -> all-gather over the mp group -> ``[tokens, out/n]``."""

    def __init__(self, in_features, out_features, weight_attr=None, has_bias=None, gather_output=True,
                 fuse_matmul_bias=False, mp_group=None, name=None):
        super().__init__()
        self.model_parallel_group = mp_group or _hcg().get_model_parallel_group()
        self.world_size = self.model_parallel_group.nranks if self.model_parallel_group else 1
        self.is_mp = self.world_size > 1
        assert gather_output is False, "sequence parallel keeps the column output sharded"
        assert out_features % self.world_size == 0
        per = out_features // self.world_size
        if self.is_mp:
            with get_rng_state_tracker().rng_state():
                self.weight = self.create_parameter([in_features, per], weight_attr)
            _mark(self.weight, 1)
        else:
            self.weight = self.create_parameter([in_features, per], weight_attr)
        self.bias = self.create_parameter([per], None, is_bias=True) if has_bias else None
        if self.bias is not None and self.is_mp:
            _mark(self.bias, 0)

    def forward(self, x):
        if not self.is_mp:
            return F.linear(x, self.weight, self.bias)
        if _use_fused(x, self.weight, self.model_parallel_group, x.shape[0]):
            from ....parallel import fused_linear
            out = fused_linear.allgather_linear(x, self.weight, self.model_parallel_group)
            return out if self.bias is None else out + self.bias
        full = as_tensor(AllGatherOp.apply(x, self.model_parallel_group))
        return F.linear(full, self.weight, self.bias)


class RowSequenceParallelLinear(Layer):
    """x: ``[tokens, in/n]`` -> GEMM -> reduce-scatter over the mp group -> ``[tokens/n, out]``."""

    def __init__(self, in_features, out_features, weight_attr=None, has_bias=True, input_is_parallel=False,
                 fuse_matmul_bias=False, mp_group=None, name=None):
        super().__init__()
        self.model_parallel_group = mp_group or _hcg().get_model_parallel_group()
        self.world_size = self.model_parallel_group.nranks if self.model_parallel_group else 1
        self.is_mp = self.world_size > 1
        assert input_is_parallel, "sequence parallel expects an already sharded input"
        assert in_features % self.world_size == 0
        per = in_features // self.world_size
        if self.is_mp:
            with get_rng_state_tracker().rng_state():
                self.weight = self.create_parameter([per, out_features], weight_attr)
            _mark(self.weight, 0)
        else:
            self.weight = self.create_parameter([per, out_features], weight_attr)
        if has_bias:
            self.bias = self.create_parameter([out_features], None, is_bias=True)
            if self.is_mp:
                mark_as_sequence_parallel_parameter(self.bias)
        else:
            self.bias = None

    def forward(self, x):
        if not self.is_mp:
            return F.linear(x, self.weight, self.bias)
        if _use_fused(x, self.weight, self.model_parallel_group, x.shape[0] // self.world_size):
            from ....parallel import fused_linear
            out = fused_linear.linear_reduce_scatter(x, self.weight, self.model_parallel_group)
        else:
            out = as_tensor(ReduceScatterOp.apply(F.linear(x, self.weight), self.model_parallel_group))
        return out if self.bias is None else out + self.bias


SPInnerOverlapLinear = ColumnSequenceParallelLinear


from ..layers.mpu.mp_layers import (MPScale, is_fused_linear_param_grad_add_supported,  # noqa: E402,F401
                                    is_fused_matmul_bias_supported)


def create_non_fused_allreduce_gradient_hook(param, accumulation_steps):
    """Hook that all-reduces ``param``'s gradient over the mp group every ``accumulation_steps`` calls."""
    g = _group()
    state = {"step": 0}

    def hook(*_):
        state["step"] += 1
        if state["step"] % accumulation_steps == 0 and g is not None and g.nranks > 1:
            mg = getattr(param, "main_grad", None)
            gr = mg if mg is not None else torch.Tensor.grad.__get__(param)
            if gr is not None:
                C.all_reduce(gr, group=g)
    return hook


def create_fused_allreduce_gradient_hook(parameter_list, accumulation_steps):
    """One hook shared by ``parameter_list``: when all of them have seen ``accumulation_steps`` backward passes their
    gradients are all-reduced over the mp group in one flattened buffer per dtype."""
    g = _group()
    params = list(parameter_list)
    state = {"step": 0, "total": len(params) * accumulation_steps}

    def hook(*_):
        state["step"] += 1
        if state["step"] < state["total"]:
            return
        state["step"] = 0
        if g is None or g.nranks == 1:
            return
        grads = []
        for p in params:
            mg = getattr(p, "main_grad", None)
            gr = mg if mg is not None else torch.Tensor.grad.__get__(p)
            if gr is not None:
                grads.append(gr)
        by_dtype = {}
        for gr in grads:
            by_dtype.setdefault(gr.dtype, []).append(gr)
        for gs in by_dtype.values():
            flat = torch.cat([x.reshape(-1) for x in gs])
            C.all_reduce(flat, group=g)
            off = 0
            for x in gs:
                x.copy_(flat[off:off + x.numel()].view_as(x))
                off += x.numel()
    return hook


def is_fused_matmul_bias_supported():
    """Whether GEMM + bias runs as one kernel (sequence_parallel_utils.py:229 asks for cuBLASLt's epilogue): here
    when the sm_100a kernel library is loadable on a GPU."""
    if not torch.cuda.is_available():
        return False
    try:
        from ....ops import _lib
        return _lib.kernels() is not None
    except Exception:
        return False
