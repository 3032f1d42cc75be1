"""Tensor-parallel layers (python/paddle/distributed/fleet/layers/mpu/mp_layers.py):
``VocabParallelEmbedding`` (:49), ``ColumnParallelLinear`` (:336, weight ``[in, out/n]``),
``RowParallelLinear`` (:543, weight ``[in/n, out]``, bias added after the reduce), ``ParallelCrossEntropy``
(:744).  Parameters carry ``is_distributed`` and ``split_axis`` so checkpoints and mp sync can tell shards
from replicated tensors (mp_layers.py:157-159,435-450,673-675)."""
from __future__ import annotations

import torch

from ....._core.tensor import as_tensor
from .....nn import functional as F
from .....nn.initializer import Constant
from .....nn.layer.layers import Layer
from .... import collective as C
from . import mp_ops
from .random import get_rng_state_tracker


def _hcg():
    from ... import fleet
    return fleet.get_hybrid_communicate_group()


def _mark(param, axis):
    param.is_distributed = True
    param.split_axis = axis


class VocabParallelEmbedding(Layer):
    def __init__(self, num_embeddings, embedding_dim, weight_attr=None, mp_group=None, name=None):
        super().__init__()
        hcg = _hcg()
        self.model_parallel_group = mp_group or hcg.get_model_parallel_group()
        self.world_size = self.model_parallel_group.nranks if self.model_parallel_group else 1
        self.rank = self.model_parallel_group.rank if self.model_parallel_group else 0
        assert num_embeddings % self.world_size == 0, "vocabulary must divide evenly over the mp group"
        self.origin_num_embeddings = num_embeddings
        per = num_embeddings // self.world_size
        self.vocab_start_index = self.rank * per
        self.is_mp = self.world_size > 1
        if self.is_mp:
            with get_rng_state_tracker().rng_state():
                self.weight = self.create_parameter([per, embedding_dim], weight_attr)
            _mark(self.weight, 0)
        else:
            self.weight = self.create_parameter([per, embedding_dim], weight_attr)

    def forward(self, x):
        if not self.is_mp:
            return F.embedding(x, self.weight)
        out = mp_ops._c_lookup_table(self.weight, x, start_index=self.vocab_start_index,
                                     vocab_size=self.origin_num_embeddings)
        return mp_ops._mp_allreduce(out, group=self.model_parallel_group)

    def forward_sequence_parallel(self, x):
        """Embedding of all tokens of ``x`` flattened to ``[T]``, returned as this rank's sequence shard ``[T / n, H]``
        (what ``ScatterOp.apply(embedding(x).reshape([T, H]))`` gives).  On GPUs with peer-mapped memory one kernel
        writes every row into the shard of the rank that owns its token; otherwise lookup, all-reduce and slice."""
        tokens = 1
        for d in x.shape:
            tokens *= int(d)
        if self.is_mp and mp_ops.fused_embedding_available(self.weight, tokens, self.model_parallel_group):
            return mp_ops.vocab_parallel_embedding_to_sequence_shard(x, self.weight, self.model_parallel_group,
                                                                     self.vocab_start_index)
        from ...utils.sequence_parallel_utils import ScatterOp
        h = self.forward(x)
        return ScatterOp.apply(h.reshape([tokens, h.shape[-1]]))


class ColumnParallelLinear(Layer):
    def __init__(self, in_features, out_features, weight_attr=None, has_bias=None, gather_output=True,
                 fuse_matmul_bias=False, mp_group=None, name=None):
        super().__init__()
        hcg = _hcg()
        self.model_parallel_group = mp_group or hcg.get_model_parallel_group()
        self.world_size = self.model_parallel_group.nranks if self.model_parallel_group else 1
        self.is_mp = self.world_size > 1
        self.gather_output = gather_output
        assert out_features % self.world_size == 0
        self.output_size_per_partition = out_features // self.world_size
        if self.is_mp:
            with get_rng_state_tracker().rng_state():
                self.weight = self.create_parameter([in_features, self.output_size_per_partition], weight_attr)
            _mark(self.weight, 1)
        else:
            self.weight = self.create_parameter([in_features, self.output_size_per_partition], weight_attr)
        if has_bias:
            self.bias = self.create_parameter([self.output_size_per_partition], None, is_bias=True)
            if self.is_mp:
                _mark(self.bias, 0)
        else:
            self.bias = None

    def forward(self, x):
        x_par = mp_ops._c_identity(x, group=self.model_parallel_group) if self.is_mp else x
        out = F.linear(x_par, self.weight, self.bias)
        if self.gather_output and self.is_mp:
            out = mp_ops._c_concat(out, group=self.model_parallel_group)
        return out


class RowParallelLinear(Layer):
    def __init__(self, in_features, out_features, weight_attr=None, has_bias=True, input_is_parallel=False,
                 fuse_matmul_bias=False, mp_group=None, name=None):
        super().__init__()
        hcg = _hcg()
        self.model_parallel_group = mp_group or hcg.get_model_parallel_group()
        self.world_size = self.model_parallel_group.nranks if self.model_parallel_group else 1
        self.is_mp = self.world_size > 1
        self.input_is_parallel = input_is_parallel
        assert in_features % self.world_size == 0
        self.input_size_per_partition = in_features // self.world_size
        if self.is_mp:
            with get_rng_state_tracker().rng_state():
                self.weight = self.create_parameter([self.input_size_per_partition, out_features], weight_attr)
            _mark(self.weight, 0)
        else:
            self.weight = self.create_parameter([self.input_size_per_partition, out_features], weight_attr)
        self.bias = self.create_parameter([out_features], None, is_bias=True) if has_bias else None

    def forward(self, x):
        if not self.input_is_parallel and self.is_mp:
            x = mp_ops._c_split(x, group=self.model_parallel_group)
        if self.is_mp and torch.is_tensor(x) and x.is_cuda:
            # training-size inputs on GPUs: the reduction runs from inside the GEMM (GEMM -> reduce-scatter kernel) and
            # an all-gather of the reduced slabs completes the all-reduce
            from .....ops import functional as K
            from .....parallel import fused_linear_impl as FL
            x2 = x.reshape([-1, x.shape[-1]])
            if K.get_kernel_policy() == "fused" and FL.linear_all_reduce_ok(x2, self.weight, self.model_parallel_group):
                out = FL.linear_all_reduce(x2, self.weight, self.model_parallel_group)
                out = out.reshape([*x.shape[:-1], out.shape[-1]])
                return out + self.bias if self.bias is not None else out
        out = F.linear(x, self.weight)
        if self.is_mp:
            out = mp_ops._mp_allreduce(out, group=self.model_parallel_group)
        return out + self.bias if self.bias is not None else out


class ParallelCrossEntropy(Layer):
    def __init__(self, mp_group=None, name=None, ignore_index=-100):
        super().__init__()
        self.model_parallel_group = mp_group or _hcg().get_model_parallel_group()
        self.ignore_index = ignore_index

    def forward(self, input, label):
        return mp_ops._c_softmax_with_cross_entropy(input, label, group=self.model_parallel_group,
                                                    ignore_index=self.ignore_index)


class MPScale(torch.autograd.Function):
    """Forward divides by the tensor-parallel degree, backward passes the gradient through (mp_layers.py ``MPScale``)."""

    @staticmethod
    def forward(ctx, x, mp_degree):
        return x / mp_degree

    @staticmethod
    def backward(ctx, dout):
        return dout, None


def is_fused_matmul_bias_supported():
    """The bias add is an epilogue of this framework's GEMM kernel whenever the GPU library is loaded."""
    return torch.cuda.is_available()


def is_fused_linear_param_grad_add_supported():
    """Weight gradients are accumulated into fp32 ``main_grad`` by the GEMM epilogue on GPU."""
    return torch.cuda.is_available()


class InnerOverlapLinear(torch.autograd.Function):
    """Column-parallel linear whose backward starts the all-reduce of the input gradient over the tensor-parallel
    group and computes the weight / bias gradients while it is in flight (mp_layers.py:190).  With
    ``mp_fused_linear_param_grad_add`` the weight gradient is accumulated straight into ``weight.main_grad``."""

    @staticmethod
    def forward(ctx, x, weight, bias, fuse_matmul_bias, mp_async_allreduce, mp_skip_c_identity,
                mp_fused_linear_param_grad_add, model_parallel_group):
        ctx.save_for_backward(x, weight)
        ctx.has_bias, ctx.group, ctx.fused_add, ctx.w_ref, ctx.b_ref = bias is not None, model_parallel_group, \
            mp_fused_linear_param_grad_add, weight, bias
        y = torch.matmul(x, weight)
        return y if bias is None else y + bias

    @staticmethod
    def backward(ctx, dy):
        from .... import collective as C
        x, weight = ctx.saved_tensors
        dx = torch.matmul(dy, weight.t())
        g = ctx.group
        task = C.all_reduce(dx, group=g, sync_op=False) if (g is not None and g.nranks > 1) else None
        x2, d2 = x.reshape(-1, x.shape[-1]), dy.reshape(-1, dy.shape[-1])
        dw = db = None
        if ctx.fused_add and getattr(ctx.w_ref, "main_grad", None) is not None:
            from .....incubate.nn.functional import fused_linear_param_grad_add
            bias_acc = getattr(ctx.b_ref, "main_grad", None) if ctx.has_bias else None
            fused_linear_param_grad_add(x2, d2, ctx.w_ref.main_grad, bias_acc, True, ctx.has_bias and bias_acc is not None)
            if ctx.has_bias and bias_acc is None:
                db = d2.sum(0)
        else:
            dw = x2.t() @ d2
            db = d2.sum(0) if ctx.has_bias else None
        if task is not None:
            task.wait()
        return dx, dw, db, None, None, None, None, None


class ParallelMultiLabelCrossEntropy(Layer):
    """Vocab-parallel cross entropy with several weighted labels per row (mp_layers.py:796)."""

    def __init__(self, mp_group=None, name=None, ignore_index=-100, sum_multi_label_loss=True):
        super().__init__()
        self.name = name
        self.model_parallel_group = mp_group
        self.ignore_index, self.sum_multi_label_loss = ignore_index, sum_multi_label_loss

    def forward(self, input, label, smooth_weight):
        return mp_ops._c_softmax_with_multi_label_cross_entropy(
            input, label, smooth_weight, group=self.model_parallel_group, ignore_index=self.ignore_index,
            sum_multi_label_loss=self.sum_multi_label_loss)
