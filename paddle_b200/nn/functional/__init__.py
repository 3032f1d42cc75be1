"""``paddle.nn.functional``.  Hot operators (linear, layer_norm, embedding, cross entropy, attention)
route to this library's sm_100a kernels through ``paddle_b200.ops.functional``; the long tail
wraps the corresponding torch operator under Paddle's argument names."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as TF

from ..._core import dtype as _dt
from ..._core.tensor import as_tensor
from ...ops import functional as K
from .flash_attention import (flash_attention, flash_attn_unpadded, flashmask_attention,  # noqa: F401
                              scaled_dot_product_attention, sdp_kernel)


# ------------------------------------------------------------------ linear / embedding
def linear(x, weight, bias=None, name=None):
    """y = x @ weight + bias with weight ``[in_features, out_features]``
    (python/paddle/nn/functional/common.py:2238)."""
    return K.linear(x, weight, bias)


def bilinear(x1, x2, weight, bias=None, name=None):
    return TF.bilinear(x1, x2, weight, None if bias is None else bias.reshape(-1))


def embedding(x, weight, padding_idx=None, max_norm=None, norm_type=2.0, sparse=False, scale_grad_by_freq=False,
              name=None):
    if padding_idx is not None and padding_idx < 0:
        padding_idx = weight.shape[0] + padding_idx
    return K.embedding(x, weight, padding_idx)


def one_hot(x, num_classes, name=None):
    return TF.one_hot(x.long(), num_classes).to(_dt.get_default_dtype())


# ------------------------------------------------------------------ activations
def relu(x, name=None):
    return TF.relu(x)


def relu_(x, name=None):
    return TF.relu_(x)


def relu6(x, name=None):
    return TF.relu6(x)


def gelu(x, approximate=False, name=None):
    return TF.gelu(x, approximate="tanh" if approximate else "none")


def silu(x, name=None):
    return TF.silu(x)


swish = silu


def sigmoid(x, name=None):
    return torch.sigmoid(x)


def tanh(x, name=None):
    return torch.tanh(x)


def leaky_relu(x, negative_slope=0.01, name=None):
    return TF.leaky_relu(x, negative_slope)


def elu(x, alpha=1.0, name=None):
    return TF.elu(x, alpha)


def selu(x, scale=1.0507009873554805, alpha=1.6732632423543772, name=None):
    return scale * TF.elu(x, alpha)


def celu(x, alpha=1.0, name=None):
    return TF.celu(x, alpha)


def prelu(x, weight, data_format="NCHW", name=None):
    return TF.prelu(x, weight)


def rrelu(x, lower=1.0 / 8.0, upper=1.0 / 3.0, training=True, name=None):
    return TF.rrelu(x, lower, upper, training)


def hardtanh(x, min=-1.0, max=1.0, name=None):
    return TF.hardtanh(x, min, max)


def hardsigmoid(x, slope=0.1666667, offset=0.5, name=None):
    return torch.clamp(x * slope + offset, 0.0, 1.0)


def hardswish(x, name=None):
    return TF.hardswish(x)


def hardshrink(x, threshold=0.5, name=None):
    return TF.hardshrink(x, threshold)


def softshrink(x, threshold=0.5, name=None):
    return TF.softshrink(x, threshold)


def tanhshrink(x, name=None):
    return x - torch.tanh(x)


def thresholded_relu(x, threshold=1.0, value=0.0, name=None):
    return torch.where(x > threshold, x, torch.full_like(x, value))


def softplus(x, beta=1.0, threshold=20.0, name=None):
    return TF.softplus(x, beta, threshold)


def softsign(x, name=None):
    return TF.softsign(x)


def mish(x, name=None):
    return TF.mish(x)


def log_sigmoid(x, name=None):
    return TF.logsigmoid(x)


def maxout(x, groups, axis=1, name=None):
    shape = list(x.shape)
    shape[axis:axis + 1] = [shape[axis] // groups, groups]
    return x.reshape(shape).amax(axis + 1)


def glu(x, axis=-1, name=None):
    return TF.glu(x, axis)


def swiglu(x, y=None, name=None):
    return K.swiglu(x, y)


def softmax(x, axis=-1, dtype=None, name=None):
    return TF.softmax(x, dim=axis, dtype=_dt.to_torch(dtype))


def log_softmax(x, axis=-1, dtype=None, name=None):
    return TF.log_softmax(x, dim=axis, dtype=_dt.to_torch(dtype))


def gumbel_softmax(x, temperature=1.0, hard=False, axis=-1, name=None):
    return TF.gumbel_softmax(x, temperature, hard, dim=axis)


# ------------------------------------------------------------------ normalisation
def layer_norm(x, normalized_shape, weight=None, bias=None, epsilon=1e-5, name=None):
    return K.layer_norm(x, normalized_shape, weight, bias, epsilon)


def rms_norm(x, weight, epsilon=1e-6):
    return K.rms_norm(x, weight, epsilon)


def batch_norm(x, running_mean, running_var, weight=None, bias=None, training=False, momentum=0.9, epsilon=1e-5,
               data_format="NCHW", use_global_stats=None, name=None):
    use_batch = training and not use_global_stats
    cl = data_format in ("NHWC", "NLC", "NDHWC")
    if cl:
        x = x.movedim(-1, 1)
    y = TF.batch_norm(x, running_mean, running_var, weight, bias, use_batch, 1.0 - momentum, epsilon)
    return y.movedim(1, -1) if cl else y


def instance_norm(x, running_mean=None, running_var=None, weight=None, bias=None, use_input_stats=True,
                  momentum=0.9, eps=1e-5, data_format="NCHW", name=None):
    return TF.instance_norm(x, running_mean, running_var, weight, bias, use_input_stats, 1.0 - momentum, eps)


def group_norm(x, num_groups, epsilon=1e-5, weight=None, bias=None, data_format="NCHW", name=None):
    if data_format == "NHWC":
        return TF.group_norm(x.movedim(-1, 1), num_groups, weight, bias, epsilon).movedim(1, -1)
    return TF.group_norm(x, num_groups, weight, bias, epsilon)


def local_response_norm(x, size, alpha=1e-4, beta=0.75, k=1.0, data_format="NCHW", name=None):
    return TF.local_response_norm(x, size, alpha, beta, k)


def normalize(x, p=2, axis=1, epsilon=1e-12, name=None):
    return TF.normalize(x, p, axis, epsilon)


# ------------------------------------------------------------------ dropout
def dropout(x, p=0.5, axis=None, training=True, mode="upscale_in_train", name=None):
    if not training:
        return x if mode == "upscale_in_train" else x * (1.0 - p)
    if p == 0.0:
        return x
    if axis is None:
        if 0.0 < p < 1.0 and K.dropout_add_supported(x):
            # own Philox kernel: keep decisions addressed by the CUDA generator's (seed, offset), regenerated in backward
            return K.dropout_add(x, None, p, mode == "upscale_in_train")[0]
        y = TF.dropout(x, p, True)
        return y if mode == "upscale_in_train" else y * (1.0 - p)
    axes = [axis] if isinstance(axis, int) else list(axis)
    mshape = [s if i in axes else 1 for i, s in enumerate(x.shape)]
    mask = (torch.rand(mshape, device=x.device) >= p).to(x.dtype)
    return x * mask / (1.0 - p) if mode == "upscale_in_train" else x * mask


def dropout2d(x, p=0.5, training=True, data_format="NCHW", name=None):
    return TF.dropout2d(x, p, training)


def dropout3d(x, p=0.5, training=True, data_format="NCDHW", name=None):
    return TF.dropout3d(x, p, training)


def alpha_dropout(x, p=0.5, training=True, name=None):
    return TF.alpha_dropout(x, p, training)


# ------------------------------------------------------------------ losses
def _reduce(loss, reduction):
    if reduction == "mean":
        return loss.mean()
    if reduction == "sum":
        return loss.sum()
    return loss


def cross_entropy(input, label, weight=None, ignore_index=-100, reduction="mean", soft_label=False, axis=-1,
                  use_softmax=True, label_smoothing=0.0, name=None):
    """python/paddle/nn/functional/loss.py ``cross_entropy``; the hard-label, softmax, last-axis case
    runs the fused softmax-CE kernel."""
    if axis not in (-1, input.dim() - 1):
        input = input.movedim(axis, -1)
        if soft_label:
            label = label.movedim(axis, -1)
    if label_smoothing > 0.0 and label.is_floating_point() and label.dim() == input.dim() and label.shape[-1] == input.shape[-1]:
        # one-hot (float) labels under label smoothing are smoothed and treated as soft labels
        label = label * (1 - label_smoothing) + label_smoothing / input.shape[-1]
        soft_label, label_smoothing = True, 0.0
    if soft_label or not use_softmax or label_smoothing > 0.0 or weight is not None:
        wide = input if input.dtype == torch.float64 else input.float()
        logp = TF.log_softmax(wide, -1) if use_softmax else torch.log(wide)
        if not soft_label:
            lab = label.squeeze(-1) if label.dim() == input.dim() else label
            if label_smoothing > 0.0:
                oh = TF.one_hot(lab.clamp(min=0).long(), input.shape[-1]).to(logp.dtype)
                oh = oh * (1 - label_smoothing) + label_smoothing / input.shape[-1]
                loss = -(oh * logp).sum(-1)
                loss = torch.where(lab == ignore_index, torch.zeros_like(loss), loss)
            else:
                loss = TF.nll_loss(logp.reshape(-1, logp.shape[-1]), lab.reshape(-1).long(), weight,
                                   ignore_index=ignore_index, reduction="none").view(lab.shape)
            if reduction == "mean":
                if weight is not None:
                    wsum = weight[lab.clamp(min=0)].masked_fill(lab == ignore_index, 0).sum()
                    return loss.sum() / wsum
                valid = (lab != ignore_index).sum().clamp(min=1)
                return loss.sum() / valid
            return _reduce(loss, reduction)
        loss = -(label.to(logp.dtype) * logp).sum(-1)
        if weight is not None:
            loss = loss * (label.to(logp.dtype) * weight.to(logp.dtype)).sum(-1)
        return _reduce(loss, reduction)
    lab = label.squeeze(-1) if label.dim() == input.dim() else label
    loss = K.softmax_cross_entropy(input, lab, ignore_index)
    if reduction == "mean":
        valid = (lab != ignore_index).sum().clamp(min=1)
        return loss.sum() / valid
    if reduction == "sum":
        return loss.sum()
    return loss.unsqueeze(-1) if label.dim() == input.dim() else loss


def softmax_with_cross_entropy(logits, label, soft_label=False, ignore_index=-100, numeric_stable_mode=True,
                               return_softmax=False, axis=-1):
    loss = cross_entropy(logits, label, ignore_index=ignore_index, reduction="none", soft_label=soft_label, axis=axis)
    if loss.dim() < logits.dim():
        loss = loss.unsqueeze(axis)
    if return_softmax:
        return loss, softmax(logits, axis)
    return loss


def nll_loss(input, label, weight=None, ignore_index=-100, reduction="mean", name=None):
    label = label.long()
    if input.dim() == 2 and label.dim() == 2 and label.shape[1] == 1:
        label = label.reshape(-1)                      # [N, 1] class ids are taken as [N]
    return TF.nll_loss(input, label, weight, ignore_index=ignore_index, reduction=reduction)


def mse_loss(input, label, reduction="mean", name=None):
    return TF.mse_loss(input, label, reduction=reduction)


def l1_loss(input, label, reduction="mean", name=None):
    return TF.l1_loss(input, label, reduction=reduction)


def smooth_l1_loss(input, label, reduction="mean", delta=1.0, name=None):
    return TF.huber_loss(input, label, reduction=reduction, delta=delta)


def binary_cross_entropy(input, label, weight=None, reduction="mean", name=None):
    return TF.binary_cross_entropy(input, label, weight, reduction=reduction)


def binary_cross_entropy_with_logits(logit, label, weight=None, reduction="mean", pos_weight=None, name=None):
    return TF.binary_cross_entropy_with_logits(logit, label, weight, reduction=reduction, pos_weight=pos_weight)


def kl_div(input, label, reduction="mean", log_target=False, name=None):
    return TF.kl_div(input, label, reduction=reduction, log_target=log_target)


def margin_ranking_loss(input, other, label, margin=0.0, reduction="mean", name=None):
    return TF.margin_ranking_loss(input, other, label, margin=margin, reduction=reduction)


def hinge_embedding_loss(input, label, margin=1.0, reduction="mean", name=None):
    return TF.hinge_embedding_loss(input, label, margin, reduction=reduction)


def cosine_embedding_loss(input1, input2, label, margin=0, reduction="mean", name=None):
    return TF.cosine_embedding_loss(input1, input2, label, margin, reduction=reduction)


def cosine_similarity(x1, x2, axis=1, eps=1e-8):
    return TF.cosine_similarity(x1, x2, axis, eps)


def pairwise_distance(x, y, p=2.0, epsilon=1e-6, keepdim=False, name=None):
    return TF.pairwise_distance(x, y, p, epsilon, keepdim)


def triplet_margin_loss(input, positive, negative, margin=1.0, p=2, epsilon=1e-6, swap=False, reduction="mean",
                        name=None):
    return TF.triplet_margin_loss(input, positive, negative, margin, p, epsilon, swap, reduction=reduction)


def sigmoid_focal_loss(logit, label, normalizer=None, alpha=0.25, gamma=2.0, reduction="sum", name=None):
    p = torch.sigmoid(logit)
    ce = TF.binary_cross_entropy_with_logits(logit, label, reduction="none")
    pt = p * label + (1 - p) * (1 - label)
    loss = ce * ((1 - pt) ** gamma) * (alpha * label + (1 - alpha) * (1 - label))
    if normalizer is not None:
        loss = loss / normalizer
    return _reduce(loss, reduction)


def ctc_loss(log_probs, labels, input_lengths, label_lengths, blank=0, reduction="mean", norm_by_times=False):
    return TF.ctc_loss(TF.log_softmax(log_probs, -1), labels, input_lengths, label_lengths, blank, reduction)


def label_smooth(label, prior_dist=None, epsilon=0.1, name=None):
    n = label.shape[-1]
    return (1 - epsilon) * label + epsilon * (prior_dist if prior_dist is not None else 1.0 / n)


def square_error_cost(input, label):
    return (input - label) ** 2


def log_loss(input, label, epsilon=1e-4, name=None):
    return -label * torch.log(input + epsilon) - (1 - label) * torch.log(1 - input + epsilon)


# ------------------------------------------------------------------ conv / pool / vision
def _tuple(v, n):
    return tuple(v) if isinstance(v, (list, tuple)) else (v,) * n


def _conv_pad(padding, n):
    if isinstance(padding, str):
        return padding.lower()
    if isinstance(padding, (list, tuple)) and len(padding) == 2 * n:
        return tuple(padding[::2])
    return _tuple(padding, n)


def conv1d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, data_format="NCL", name=None):
    if data_format == "NLC":
        return TF.conv1d(x.transpose(1, 2), weight, bias, stride, _conv_pad(padding, 1), dilation, groups).transpose(1, 2)
    return TF.conv1d(x, weight, bias, stride, _conv_pad(padding, 1), dilation, groups)


def conv2d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, data_format="NCHW", name=None):
    if data_format == "NHWC":
        return TF.conv2d(x.permute(0, 3, 1, 2), weight, bias, stride, _conv_pad(padding, 2), dilation, groups).permute(0, 2, 3, 1)
    return TF.conv2d(x, weight, bias, stride, _conv_pad(padding, 2), dilation, groups)


def conv3d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, data_format="NCDHW", name=None):
    return TF.conv3d(x, weight, bias, stride, _conv_pad(padding, 3), dilation, groups)


def conv1d_transpose(x, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1,
                     output_size=None, data_format="NCL", name=None):
    return TF.conv_transpose1d(x, weight, bias, stride, _conv_pad(padding, 1), output_padding, groups, dilation)


def conv2d_transpose(x, weight, bias=None, stride=1, padding=0, output_padding=0, dilation=1, groups=1,
                     output_size=None, data_format="NCHW", name=None):
    return TF.conv_transpose2d(x, weight, bias, stride, _conv_pad(padding, 2), output_padding, groups, dilation)


def conv3d_transpose(x, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1,
                     output_size=None, data_format="NCDHW", name=None):
    return TF.conv_transpose3d(x, weight, bias, stride, _conv_pad(padding, 3), output_padding, groups, dilation)


def max_pool1d(x, kernel_size, stride=None, padding=0, return_mask=False, ceil_mode=False, name=None):
    return TF.max_pool1d(x, kernel_size, stride, padding, 1, ceil_mode, return_mask)


def max_pool2d(x, kernel_size, stride=None, padding=0, return_mask=False, ceil_mode=False, data_format="NCHW",
               name=None):
    return TF.max_pool2d(x, kernel_size, stride, padding, 1, ceil_mode, return_mask)


def max_pool3d(x, kernel_size, stride=None, padding=0, return_mask=False, ceil_mode=False, data_format="NCDHW",
               name=None):
    return TF.max_pool3d(x, kernel_size, stride, padding, 1, ceil_mode, return_mask)


def avg_pool1d(x, kernel_size, stride=None, padding=0, exclusive=True, ceil_mode=False, name=None):
    return TF.avg_pool1d(x, kernel_size, stride, padding, ceil_mode, not exclusive)


def avg_pool2d(x, kernel_size, stride=None, padding=0, ceil_mode=False, exclusive=True, divisor_override=None,
               data_format="NCHW", name=None):
    return TF.avg_pool2d(x, kernel_size, stride, padding, ceil_mode, not exclusive, divisor_override)


def avg_pool3d(x, kernel_size, stride=None, padding=0, ceil_mode=False, exclusive=True, divisor_override=None,
               data_format="NCDHW", name=None):
    return TF.avg_pool3d(x, kernel_size, stride, padding, ceil_mode, not exclusive, divisor_override)


def adaptive_avg_pool1d(x, output_size, name=None):
    return TF.adaptive_avg_pool1d(x, output_size)


def adaptive_avg_pool2d(x, output_size, data_format="NCHW", name=None):
    return TF.adaptive_avg_pool2d(x, output_size)


def adaptive_avg_pool3d(x, output_size, data_format="NCDHW", name=None):
    return TF.adaptive_avg_pool3d(x, output_size)


def adaptive_max_pool1d(x, output_size, return_mask=False, name=None):
    return TF.adaptive_max_pool1d(x, output_size, return_mask)


def adaptive_max_pool2d(x, output_size, return_mask=False, name=None):
    return TF.adaptive_max_pool2d(x, output_size, return_mask)


def pad(x, pad, mode="constant", value=0.0, data_format=None, pad_from_left_axis=True, name=None):
    pad = [int(p) for p in (pad.tolist() if isinstance(pad, torch.Tensor) else pad)]
    nd = x.dim()
    if data_format is None:
        data_format = {3: "NCL", 4: "NCHW", 5: "NCDHW"}.get(nd, "NCHW")
    if len(pad) == 2 * nd and mode == "constant":
        # per-axis pairs; from the first axis by default (torch wants the last axis first), from the last one otherwise
        pairs = [pad[2 * i:2 * i + 2] for i in range(nd)]
        flat = [v for pr in reversed(pairs) for v in pr] if pad_from_left_axis else list(pad)
        return TF.pad(x, flat, mode=mode, value=value) if mode == "constant" else TF.pad(x, flat, mode=mode)
    cl = data_format in ("NHWC", "NLC", "NDHWC")
    if cl:
        x = x.movedim(-1, 1)
    tmode = {"constant": "constant", "reflect": "reflect", "replicate": "replicate", "circular": "circular"}[mode]
    y = TF.pad(x, pad, mode=tmode, value=value) if tmode == "constant" else TF.pad(x, pad, mode=tmode)
    return y.movedim(1, -1) if cl else y


def zeropad2d(x, padding, data_format="NCHW", name=None):
    return pad(x, padding, "constant", 0.0, data_format)


def interpolate(x, size=None, scale_factor=None, mode="nearest", align_corners=False, align_mode=0,
                data_format="NCHW", name=None):
    if isinstance(size, torch.Tensor):
        size = size.tolist()
    kw = {}
    if mode in ("linear", "bilinear", "bicubic", "trilinear"):
        kw["align_corners"] = align_corners
    cl = data_format in ("NHWC", "NLC", "NDHWC")
    if cl:
        x = x.movedim(-1, 1)
    y = TF.interpolate(x, size=size, scale_factor=scale_factor, mode=mode, **kw)
    return y.movedim(1, -1) if cl else y


upsample = interpolate


def grid_sample(x, grid, mode="bilinear", padding_mode="zeros", align_corners=True, name=None):
    return TF.grid_sample(x, grid, mode, padding_mode, align_corners)


def affine_grid(theta, out_shape, align_corners=True, name=None):
    return TF.affine_grid(theta, list(out_shape), align_corners)


def pixel_shuffle(x, upscale_factor, data_format="NCHW", name=None):
    return TF.pixel_shuffle(x, upscale_factor)


def pixel_unshuffle(x, downscale_factor, data_format="NCHW", name=None):
    return TF.pixel_unshuffle(x, downscale_factor)


def channel_shuffle(x, groups, data_format="NCHW", name=None):
    return TF.channel_shuffle(x, groups)


def unfold(x, kernel_sizes, strides=1, paddings=0, dilations=1, name=None):
    return TF.unfold(x, kernel_sizes, dilations, paddings, strides)


def fold(x, output_sizes, kernel_sizes, strides=1, paddings=0, dilations=1, name=None):
    return TF.fold(x, output_sizes, kernel_sizes, dilations, paddings, strides)


def sequence_mask(x, maxlen=None, dtype="int64", name=None):
    maxlen = int(x.max().item()) if maxlen is None else maxlen
    return (torch.arange(maxlen, device=x.device)[None, :] < x.unsqueeze(-1)).to(_dt.to_torch(dtype))


def temporal_shift(x, seg_num, shift_ratio=0.25, name=None, data_format="NCHW"):
    nt, c, h, w = x.shape
    x5 = x.reshape(nt // seg_num, seg_num, c, h, w)
    c1, c2 = int(c * shift_ratio), int(c * 2 * shift_ratio)
    out = torch.zeros_like(x5)
    out[:, :-1, :c1] = x5[:, 1:, :c1]
    out[:, 1:, c1:c2] = x5[:, :-1, c1:c2]
    out[:, :, c2:] = x5[:, :, c2:]
    return out.reshape(nt, c, h, w)


from .extras import *  # noqa: E402,F401,F403
from .extras import (elu_, hardtanh_, leaky_relu_, softmax_, tanh_, thresholded_relu_)  # noqa: E402,F401


from ..._core.submodule_alias import alias_submodules as _alias  # noqa: E402
_alias(__name__, ("loss", "activation", "common", "conv", "distance", "extension", "input", "norm", "pooling", "sparse_attention", "vision"))
# ``F.flash_attention`` is a module in the reference and a function here: the function carries the module's names
for _n in ("flash_attention", "flash_attn_unpadded", "flashmask_attention", "scaled_dot_product_attention", "flash_attn_qkvpacked",
           "flash_attn_varlen_qkvpacked", "flash_attn_varlen_func", "flash_attention_with_sparse_mask", "sdp_kernel", "calc_reduced_attention_scores"):
    if _n in globals():
        setattr(flash_attention, _n, globals()[_n])
del _n
