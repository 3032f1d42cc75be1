"""``paddle.incubate.layers`` (python/paddle/incubate/layers/nn.py): functional layers of recommender models."""
from __future__ import annotations

import torch

from ..._core.tensor import as_tensor

__all__ = []


def _p(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


def shuffle_batch(x, seed=None):
    """Random permutation of the rows of ``x`` (all leading dimensions flattened)."""
    t = _p(x)
    rows = t.reshape(-1, t.shape[-1])
    g = torch.Generator(device="cpu")
    if seed is not None:
        g.manual_seed(int(seed))
    else:
        g.seed()
    return as_tensor(rows[torch.randperm(rows.shape[0], generator=g).to(t.device)].reshape(t.shape))


def _slice_cols(t, start_index, length):
    start = start_index if start_index >= 0 else t.shape[1] + start_index
    end = t.shape[1] if length < 0 else start + length
    return t[:, start:end]


def partial_concat(input, start_index=0, length=-1):
    return as_tensor(torch.cat([_slice_cols(_p(t), start_index, length) for t in input], 1))


def partial_sum(input, start_index=0, length=-1):
    return as_tensor(sum(_slice_cols(_p(t), start_index, length) for t in input))


def batch_fc(input, param_size, param_attr, bias_size, bias_attr, act=None):
    """Per-slot fully connected: ``out[s] = input[s] @ W[s] + b[s]`` for ``input`` [slots, batch, in]."""
    from ...nn.layer.layers import Layer
    from ...nn import functional as F
    holder = Layer()
    w = holder.create_parameter(list(param_size), param_attr, input.dtype)
    b = holder.create_parameter(list(bias_size), bias_attr, input.dtype, is_bias=True)
    out = torch.baddbmm(_p(b).reshape(b.shape[0], 1, -1), _p(input), _p(w))
    out = as_tensor(out)
    return getattr(F, act)(out) if act else out


def fused_embedding_seq_pool(input, size, is_sparse=False, padding_idx=None, combiner="sum", param_attr=None,
                             dtype="float32"):
    """Embedding lookup followed by a sum over the sequence dimension of a padded ``[batch, seq]`` id tensor."""
    from ...nn.layer.layers import Layer
    w = Layer().create_parameter(list(size), param_attr, dtype)
    ids = _p(input).long()
    if ids.dim() == 3 and ids.shape[-1] == 1:
        ids = ids[..., 0]
    emb = torch.nn.functional.embedding(ids, _p(w), padding_idx=padding_idx)
    return as_tensor(emb.sum(1))


def fused_bn_add_act(x, y, momentum=0.9, epsilon=1e-05, param_attr=None, bias_attr=None, moving_mean_name=None,
                     moving_variance_name=None, act=None, name=None):
    """``act(batch_norm(x) + y)`` for NHWC inputs."""
    from ... import nn
    from ...nn import functional as F
    bn = nn.BatchNorm2D(x.shape[-1], momentum=momentum, epsilon=epsilon, weight_attr=param_attr, bias_attr=bias_attr,
                        data_format="NHWC")
    out = bn(x) + y
    return getattr(F, act or "relu")(out)


def pow2_decay_with_linear_warmup(warmup_steps, total_steps, base_lr, end_lr, dtype="float32", name=None):
    """Learning-rate schedule object: linear warm-up to ``base_lr`` then ``(base_lr - end_lr) * (1 - t)^2 + end_lr``."""
    from ...optimizer.lr import LRScheduler
    if warmup_steps > total_steps:
        raise ValueError("warmup_steps cannot be larger than total_steps")

    class _Pow2(LRScheduler):
        def get_lr(self):
            step = self.last_epoch + 1
            if step <= warmup_steps:
                return base_lr * step / warmup_steps
            if step >= total_steps:
                return end_lr
            f = 1.0 - (step - warmup_steps) / float(total_steps - warmup_steps)
            return (base_lr - end_lr) * f * f + end_lr
    return _Pow2(base_lr)
