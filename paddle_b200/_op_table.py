"""Second tier of the operator registry behind ``paddle._C_ops``: kernel-level operator names of the reference's YAML
tables (paddle/phi/ops/yaml/ops.yaml, fused_ops.yaml) that have no same-named public function.  Each entry is either
an alias to the public function of this package that implements it, or a small implementation with the operator's
kernel-level argument order (the functional forms of the optimizer updates, loss-scaling bookkeeping, the ``*_interp``
family, pooling with explicit kernel arguments, fills and random fills, views ...).  Operators of back ends that are not
built (XPU, oneDNN-only fusions, parameter-server tables) are listed in ``NOT_BUILT`` and raise with that reason."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as TF

ALIASES = {
    "accuracy": "paddle_b200.metric.accuracy",
    "all_to_all": "paddle_b200.distributed.alltoall",
    "barrier": "paddle_b200.distributed.barrier",
    "broadcast": "paddle_b200.distributed.broadcast",
    "reduce": "paddle_b200.distributed.reduce",
    "c_allreduce_sum": "paddle_b200.distributed.all_reduce",
    "c_scatter": "paddle_b200.distributed.scatter",
    "batch_fc": "paddle_b200.incubate.layers.batch_fc",
    "partial_concat": "paddle_b200.incubate.layers.partial_concat",
    "partial_sum": "paddle_b200.incubate.layers.partial_sum",
    "shuffle_batch": "paddle_b200.incubate.layers.shuffle_batch",
    "blha_get_max_len": "paddle_b200.incubate.nn.functional.blha_get_max_len",
    "block_multihead_attention_": "paddle_b200.incubate.nn.functional.block_multihead_attention",
    "masked_multihead_attention_": "paddle_b200.incubate.nn.functional.masked_multihead_attention",
    "variable_length_memory_efficient_attention":
        "paddle_b200.incubate.nn.functional.variable_length_memory_efficient_attention",
    "fused_bias_act": "paddle_b200.incubate.nn.functional.fused_bias_act",
    "fused_bias_dropout_residual_layer_norm":
        "paddle_b200.incubate.nn.functional.fused_bias_dropout_residual_layer_norm",
    "fused_bias_residual_layernorm": "paddle_b200.incubate.nn.functional.fused_layer_norm",
    "fused_dropout_add": "paddle_b200.incubate.nn.functional.fused_dropout_add",
    "fused_moe": "paddle_b200.incubate.nn.functional.fused_moe",
    "moe_dispatch": "paddle_b200.incubate.nn.functional.moe_dispatch",
    "moe_ffn": "paddle_b200.incubate.nn.functional.moe_ffn",
    "moe_reduce": "paddle_b200.incubate.nn.functional.moe_reduce",
    "gemm_epilogue": "paddle_b200.incubate.nn.functional.fused_linear_activation",
    "fc": "paddle_b200.incubate.nn.functional.fused_linear",
    "fp8_fp8_half_gemm_fused": "paddle_b200.linalg.fp8_fp8_half_gemm_fused",
    "svdvals": "paddle_b200.linalg.svdvals",
    "box_coder": "paddle_b200.vision.ops.box_coder",
    "decode_jpeg": "paddle_b200.vision.ops.decode_jpeg",
    "read_file": "paddle_b200.vision.ops.read_file",
    "generate_proposals": "paddle_b200.vision.ops.generate_proposals",
    "matrix_nms": "paddle_b200.vision.ops.matrix_nms",
    "nms": "paddle_b200.vision.ops.nms",
    "prior_box": "paddle_b200.vision.ops.prior_box",
    "psroi_pool": "paddle_b200.vision.ops.psroi_pool",
    "roi_align": "paddle_b200.vision.ops.roi_align",
    "roi_pool": "paddle_b200.vision.ops.roi_pool",
    "yolo_box": "paddle_b200.vision.ops.yolo_box",
    "yolo_loss": "paddle_b200.vision.ops.yolo_loss",
    "deformable_conv": "paddle_b200.vision.ops.deform_conv2d",
    "graph_khop_sampler": "paddle_b200.incubate.graph_khop_sampler",
    "graph_sample_neighbors": "paddle_b200.incubate.graph_sample_neighbors",
    "identity_loss": "paddle_b200.incubate.identity_loss",
    "reindex_graph": "paddle_b200.geometric.reindex_graph",
    "send_u_recv": "paddle_b200.geometric.send_u_recv",
    "send_ue_recv": "paddle_b200.geometric.send_ue_recv",
    "send_uv": "paddle_b200.geometric.send_uv",
    "weighted_sample_neighbors": "paddle_b200.geometric.weighted_sample_neighbors",
    "llm_int8_linear": "paddle_b200.nn.quant.llm_int8_linear",
    "weight_dequantize": "paddle_b200.nn.quant.weight_dequantize",
    "weight_only_linear": "paddle_b200.nn.quant.weight_only_linear",
    "weight_quantize": "paddle_b200.nn.quant.weight_quantize",
    "spectral_norm": "paddle_b200.nn.utils.spectral_norm",
    "stft": "paddle_b200.signal.stft",
    "viterbi_decode": "paddle_b200.text.viterbi_decode",
    "logsigmoid": "paddle_b200.nn.functional.log_sigmoid",
    "tanh_shrink": "paddle_b200.nn.functional.tanhshrink",
    "bce_loss": "paddle_b200.nn.functional.binary_cross_entropy",
    "kldiv_loss": "paddle_b200.nn.functional.kl_div",
    "sigmoid_cross_entropy_with_logits": "paddle_b200.nn.functional.binary_cross_entropy_with_logits",
    "pad3d": "paddle_b200.nn.functional.pad",
    "unpool": "paddle_b200.nn.functional.max_unpool2d",
    "unpool3d": "paddle_b200.nn.functional.max_unpool3d",
    "warpctc": "paddle_b200.nn.functional.ctc_loss",
    "warprnnt": "paddle_b200.nn.functional.rnnt_loss",
    "fused_softmax_mask": "paddle_b200.incubate.softmax_mask_fuse",
    "fused_softmax_mask_upper_triangle": "paddle_b200.incubate.softmax_mask_fuse_upper_triangle",
    "segment_pool": "paddle_b200.geometric.segment_sum",
    "dirichlet": "paddle_b200.distribution.Dirichlet",
    "auc": "paddle_b200.metric.Auc",
}

NOT_BUILT = {
    # XPU (Kunlun) fusions
    **{n: "XPU back end" for n in (
        "add_act_xpu add_layernorm_xpu addcmul_xpu block_multihead_attention_xpu bn_act_xpu conv1d_xpu conv2d_transpose_xpu "
        "conv2d_xpu cross_attention_xpu dequantize_xpu embedding_with_eltwise_add_xpu fast_layernorm_xpu fast_where_xpu "
        "fc_xpu fused_multi_transformer_int8_xpu fused_multi_transformer_xpu generate_sequence_xpu group_norm_silu_xpu "
        "layer_norm_act_xpu layer_norm_relu_xpu mask_adaptive_xpu multi_encoder_xpu pad2d_xpu qkv_attention_xpu quantize_xpu "
        "roformer_relative_embedding_xpu sequence_unpad_xpu sine_pos_xpu spatial_transformer_resblock_xpu "
        "weight_only_linear_xpu yolo_box_xpu npu_identity").split()},
    # oneDNN / CPU inference graph fusions and LoD sequence kernels of the legacy stack
    **{n: "legacy CPU inference fusion (LoD sequence kernels)" for n in (
        "attention_lstm fused_embedding_fc_lstm fusion_gru fusion_lstm fusion_repeated_fc_relu fusion_seqconv_eltadd_relu "
        "fusion_seqpool_concat fusion_seqpool_cvm_concat fusion_squared_mat_sub fusion_transpose_flatten_concat "
        "fusion_group fused_seqpool_cvm sequence_conv sequence_pool im2sequence match_matrix_tensor pyramid_hash "
        "rank_attention crf_decoding ctc_align chunk_eval beam_search lookup_table_dequant self_dp_attention "
        "multihead_matmul qkv_unpack_mha fused_token_prune").split()},
    # parameter-server / recommendation tables and DGC
    **{n: "parameter-server stack" for n in "cvm tdm_child tdm_sampler dgc dgc_clip_by_norm dgc_momentum dpsgd".split()},
    # cuDNN v8 fused conv-bn graph ops
    **{n: "cuDNN fused conv/bn graph operator" for n in (
        "fused_dconv_drelu_dbn fused_scale_bias_add_relu fused_scale_bias_relu_conv_bn resnet_basic_block resnet_unit "
        "squeeze_excitation_block fused_conv2d_add_act fused_batch_norm_act fused_bn_add_activation "
        "distributed_fused_lamb_init").split()},
}


def _t(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else x


def _wrap(x):
    from ._core.tensor import as_tensor
    if isinstance(x, torch.Tensor):
        return as_tensor(x)
    if isinstance(x, (tuple, list)):
        return type(x)(_wrap(v) for v in x)
    return x


# ------------------------------------------------------------------------------------------------ optimizer updates
# Functional forms with the YAML argument order (param, grad, learning_rate, state..., master_param, hyper-parameters);
# they update in place and return the updated tensors, like the reference's inplace (`_`) operators.
def sgd_(param, learning_rate, grad, master_param=None, multi_precision=False):
    p = master_param if (multi_precision and master_param is not None) else param
    _t(p).add_(_t(grad).to(p.dtype) * (-float(learning_rate)))
    if p is not param:
        _t(param).copy_(_t(p))
    return param, master_param


def momentum_(param, grad, velocity, learning_rate, master_param=None, mu=0.9, use_nesterov=False,
              regularization_method="", regularization_coeff=0.0, multi_precision=False, rescale_grad=1.0):
    p = master_param if (multi_precision and master_param is not None) else param
    g = _t(grad).to(p.dtype) * rescale_grad
    if regularization_method == "l2_decay":
        g = g + regularization_coeff * _t(p)
    v = _t(velocity)
    v.mul_(mu).add_(g)
    lr = float(learning_rate)
    _t(p).add_((g + mu * v) * -lr if use_nesterov else v * -lr)
    if p is not param:
        _t(param).copy_(_t(p))
    return param, velocity, master_param


def _adam_core(param, grad, lr, m1, m2, b1p, b2p, master, beta1, beta2, eps, coeff, decoupled, multi_precision):
    p = master if (multi_precision and master is not None) else param
    g = _t(grad).to(torch.float32)
    w = _t(p).to(torch.float32)
    lr = float(lr)
    if decoupled and coeff:
        w = w * (1.0 - lr * coeff)
    m, v = _t(m1), _t(m2)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    b1, b2 = float(_t(b1p).reshape(-1)[0]), float(_t(b2p).reshape(-1)[0])
    denom = v.sqrt() / math.sqrt(1 - b2) + eps
    w = w - (lr / (1 - b1)) * (m / denom)
    _t(p).copy_(w.to(p.dtype))
    _t(b1p).mul_(beta1)
    _t(b2p).mul_(beta2)
    if p is not param:
        _t(param).copy_(_t(p))
    return param, m1, m2, b1p, b2p, master


def adam_(param, grad, learning_rate, moment1, moment2, moment2_max, beta1_pow, beta2_pow, master_param=None,
          skip_update=None, beta1=0.9, beta2=0.999, epsilon=1e-8, lazy_mode=False, min_row_size_to_use_multithread=1000,
          multi_precision=False, use_global_beta_pow=False, amsgrad=False):
    if skip_update is not None and bool(_t(skip_update).reshape(-1)[0]):
        return param, moment1, moment2, moment2_max, beta1_pow, beta2_pow, master_param
    r = _adam_core(param, grad, learning_rate, moment1, moment2, beta1_pow, beta2_pow, master_param, float(beta1),
                   float(beta2), float(epsilon), 0.0, False, multi_precision)
    return r[0], r[1], r[2], moment2_max, r[3], r[4], r[5]


def adamw_(param, grad, learning_rate, moment1, moment2, moment2_max, beta1_pow, beta2_pow, master_param=None,
           skip_update=None, beta1=0.9, beta2=0.999, epsilon=1e-8, lr_ratio=1.0, coeff=0.01, with_decay=False,
           lazy_mode=False, min_row_size_to_use_multithread=1000, multi_precision=False, use_global_beta_pow=False,
           amsgrad=False):
    if skip_update is not None and bool(_t(skip_update).reshape(-1)[0]):
        return param, moment1, moment2, moment2_max, beta1_pow, beta2_pow, master_param
    r = _adam_core(param, grad, float(learning_rate) * lr_ratio, moment1, moment2, beta1_pow, beta2_pow, master_param,
                   float(beta1), float(beta2), float(epsilon), float(coeff) if with_decay else 0.0, True, multi_precision)
    return r[0], r[1], r[2], moment2_max, r[3], r[4], r[5]


def adagrad_(param, grad, moment, learning_rate, master_param=None, epsilon=1e-6, multi_precision=False):
    g = _t(grad).to(torch.float32)
    _t(moment).add_(g * g)
    _t(param).add_((-float(learning_rate) * g / (_t(moment).sqrt() + epsilon)).to(param.dtype))
    return param, moment, master_param


def rmsprop_(param, mean_square, grad, moment, learning_rate, mean_grad=None, master_param=None, epsilon=1e-10,
             decay=0.9, momentum=0.0, centered=False, multi_precision=False):
    g = _t(grad).to(torch.float32)
    ms = _t(mean_square)
    ms.mul_(decay).addcmul_(g, g, value=1 - decay)
    if centered and mean_grad is not None:
        mg = _t(mean_grad)
        mg.mul_(decay).add_(g, alpha=1 - decay)
        denom = (ms - mg * mg + epsilon).sqrt()
    else:
        denom = (ms + epsilon).sqrt()
    mom = _t(moment)
    mom.mul_(momentum).add_(float(learning_rate) * g / denom)
    _t(param).sub_(mom.to(param.dtype))
    return param, moment, mean_square, mean_grad, master_param


def adamax_(param, grad, learning_rate, moment, inf_norm, beta1_pow, master_param=None, beta1=0.9, beta2=0.999,
            epsilon=1e-8, multi_precision=False):
    g = _t(grad).to(torch.float32)
    _t(moment).mul_(beta1).add_(g, alpha=1 - beta1)
    torch.maximum(_t(inf_norm) * beta2, g.abs() + epsilon, out=_t(inf_norm))
    lr_t = float(learning_rate) / (1 - float(_t(beta1_pow).reshape(-1)[0]))
    _t(param).sub_((lr_t * _t(moment) / _t(inf_norm)).to(param.dtype))
    return param, moment, inf_norm, master_param


def adadelta_(param, grad, avg_squared_grad, avg_squared_update, learning_rate, master_param=None, rho=0.95,
              epsilon=1e-6, multi_precision=False):
    g = _t(grad).to(torch.float32)
    asg, asu = _t(avg_squared_grad), _t(avg_squared_update)
    asg.mul_(rho).addcmul_(g, g, value=1 - rho)
    upd = -((asu + epsilon) / (asg + epsilon)).sqrt() * g
    asu.mul_(rho).addcmul_(upd, upd, value=1 - rho)
    _t(param).add_((float(learning_rate) * upd).to(param.dtype))
    return param, avg_squared_grad, avg_squared_update, master_param


def lamb_(param, grad, learning_rate, moment1, moment2, beta1_pow, beta2_pow, master_param=None, skip_update=None,
          weight_decay=0.01, beta1=0.9, beta2=0.999, epsilon=1e-6, always_adapt=False, multi_precision=False):
    if skip_update is not None and bool(_t(skip_update).reshape(-1)[0]):
        return param, moment1, moment2, beta1_pow, beta2_pow, master_param
    p = master_param if (multi_precision and master_param is not None) else param
    g, w = _t(grad).to(torch.float32), _t(p).to(torch.float32)
    m, v = _t(moment1), _t(moment2)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    b1, b2 = float(_t(beta1_pow).reshape(-1)[0]), float(_t(beta2_pow).reshape(-1)[0])
    r = (m / (1 - b1)) / ((v / (1 - b2)).sqrt() + epsilon) + weight_decay * w
    wn, rn = w.norm(), r.norm()
    trust = torch.where((wn > 0) & (rn > 0), wn / rn, torch.ones_like(wn))
    _t(p).copy_((w - float(learning_rate) * trust * r).to(p.dtype))
    _t(beta1_pow).mul_(beta1)
    _t(beta2_pow).mul_(beta2)
    if p is not param:
        _t(param).copy_(_t(p))
    return param, moment1, moment2, beta1_pow, beta2_pow, master_param


# ------------------------------------------------------------------------------------------------ AMP bookkeeping
def check_finite_and_unscale_(x, scale):
    """xs /= scale; found_infinite = any non-finite value (check_finite_and_unscale_kernel.cu)."""
    inv = 1.0 / _t(scale).to(torch.float32).reshape(-1)[0]
    found = torch.zeros(1, dtype=torch.bool, device=_t(x[0]).device if x else "cpu")
    for t in x:
        tt = _t(t)
        found |= ~torch.isfinite(tt).all()
        tt.mul_(inv.to(tt.dtype))
    return x, _wrap(found)


def update_loss_scaling_(x, found_infinite, prev_loss_scaling, in_good_steps, in_bad_steps, incr_every_n_steps,
                         decr_every_n_nan_or_inf, incr_ratio, decr_ratio, stop_update=False):
    """Dynamic loss-scale state machine (update_loss_scaling_kernel.cu): after `decr_every_n_nan_or_inf` consecutive bad
    steps the scale shrinks, after `incr_every_n_steps` good ones it grows; gradients of a bad step are zeroed."""
    bad = bool(_t(found_infinite).reshape(-1)[0])
    scale, good, badn = _t(prev_loss_scaling), _t(in_good_steps), _t(in_bad_steps)
    if bad:
        for t in x:
            _t(t).zero_()
    if not stop_update:
        if bad:
            good.zero_()
            badn.add_(1)
            if int(badn.reshape(-1)[0]) >= decr_every_n_nan_or_inf:
                scale.copy_(torch.clamp(scale * decr_ratio, min=1.0))
                badn.zero_()
        else:
            badn.zero_()
            good.add_(1)
            if int(good.reshape(-1)[0]) >= incr_every_n_steps:
                grown = scale * incr_ratio
                scale.copy_(torch.where(torch.isfinite(grown), grown, scale))
                good.zero_()
    return x, prev_loss_scaling, in_good_steps, in_bad_steps


def squared_l2_norm(x):
    return _wrap(_t(x).float().pow(2).sum().reshape(1))


def clip_by_norm(x, max_norm):
    t = _t(x)
    n = t.float().norm()
    return _wrap(torch.where(n > max_norm, (t.float() * (max_norm / n)).to(t.dtype), t))


def check_numerics(tensor, op_type="", var_name="", check_nan_inf_level=0, stack_height_limit=-1, output_dir=""):
    t = _t(tensor).float()
    stats = torch.stack([torch.isnan(t).sum(), torch.isinf(t).sum(), (t == 0).sum()]).to(torch.int64)
    vals = torch.stack([t.max(), t.min(), t.mean()]) if t.numel() else torch.zeros(3)
    if check_nan_inf_level == 0 and int(stats[0] + stats[1]) > 0:
        raise RuntimeError(f"There are NAN or INF (num_nan={int(stats[0])}, num_inf={int(stats[1])}) in "
                           f"[op={op_type}] [tensor={var_name}]")
    return _wrap(stats), _wrap(vals)


# ------------------------------------------------------------------------------------------------ interpolation / pooling
def _interp(mode):
    def op(x, out_size=None, size_tensor=None, scale_tensor=None, data_format="NCHW", out_d=0, out_h=0, out_w=0, scale=(),
           interp_method=mode, align_corners=True, align_mode=1):
        t = _t(x)
        spatial = t.dim() - 2
        size = [v for v in (out_d, out_h, out_w)[3 - spatial:] if v and v > 0]
        kw = {}
        if len(size) == spatial:
            kw["size"] = size
        elif scale:
            kw["scale_factor"] = [float(s) for s in scale]
        elif out_size is not None:
            kw["size"] = [int(v) for v in _t(out_size).reshape(-1).tolist()]
        if mode != "nearest":
            kw["align_corners"] = bool(align_corners)
        return _wrap(TF.interpolate(t, mode=mode, **kw))
    return op


bilinear_interp, nearest_interp, bicubic_interp = _interp("bilinear"), _interp("nearest"), _interp("bicubic")
trilinear_interp, linear_interp = _interp("trilinear"), _interp("linear")


def _pool(nd):
    def op(x, kernel_size, strides, paddings, ceil_mode=False, exclusive=True, data_format="NCHW", pooling_type="max",
           global_pooling=False, adaptive=False, padding_algorithm="EXPLICIT"):
        t = _t(x)
        if global_pooling:
            kernel_size, paddings = list(t.shape[2:]), [0] * nd
        pads = list(paddings)[:nd] if len(paddings) == nd else list(paddings)[::2]
        if adaptive:
            f = {("max", 2): TF.adaptive_max_pool2d, ("avg", 2): TF.adaptive_avg_pool2d, ("max", 3): TF.adaptive_max_pool3d,
                 ("avg", 3): TF.adaptive_avg_pool3d}[(pooling_type, nd)]
            return _wrap(f(t, list(kernel_size)))
        if pooling_type == "max":
            f = TF.max_pool2d if nd == 2 else TF.max_pool3d
            return _wrap(f(t, list(kernel_size), list(strides), pads, ceil_mode=ceil_mode))
        f = TF.avg_pool2d if nd == 2 else TF.avg_pool3d
        return _wrap(f(t, list(kernel_size), list(strides), pads, ceil_mode=ceil_mode, count_include_pad=not exclusive))
    return op


pool2d, pool3d = _pool(2), _pool(3)


def max_pool2d_with_index(x, kernel_size, strides=(1, 1), paddings=(0, 0), global_pooling=False, adaptive=False,
                          ceil_mode=False):
    t = _t(x)
    if adaptive:
        return _wrap(TF.adaptive_max_pool2d(t, list(kernel_size), return_indices=True))
    if global_pooling:
        kernel_size, paddings = list(t.shape[2:]), [0, 0]
    return _wrap(TF.max_pool2d(t, list(kernel_size), list(strides), list(paddings), ceil_mode=ceil_mode, return_indices=True))


def max_pool3d_with_index(x, kernel_size, strides=(1, 1, 1), paddings=(0, 0, 0), global_pooling=False, adaptive=False,
                          ceil_mode=False):
    t = _t(x)
    if adaptive:
        return _wrap(TF.adaptive_max_pool3d(t, list(kernel_size), return_indices=True))
    if global_pooling:
        kernel_size, paddings = list(t.shape[2:]), [0, 0, 0]
    return _wrap(TF.max_pool3d(t, list(kernel_size), list(strides), list(paddings), ceil_mode=ceil_mode, return_indices=True))


max_pool2d_v2 = max_pool2d_with_index


def depthwise_conv2d(input, filter, strides=(1, 1), paddings=(0, 0), padding_algorithm="EXPLICIT", groups=1,
                     dilations=(1, 1), data_format="NCHW"):
    t = _t(input)
    return _wrap(TF.conv2d(t, _t(filter), None, list(strides), list(paddings)[:2], list(dilations), t.shape[1]))


def depthwise_conv2d_transpose(x, filter, strides=(1, 1), paddings=(0, 0), output_padding=(), output_size=(),
                               padding_algorithm="EXPLICIT", groups=1, dilations=(1, 1), data_format="NCHW"):
    t = _t(x)
    return _wrap(TF.conv_transpose2d(t, _t(filter), None, list(strides), list(paddings)[:2],
                                     list(output_padding) or 0, t.shape[1], list(dilations)))


def conv2d_transpose_bias(x, filter, bias, strides=(1, 1), paddings=(0, 0), output_padding=(), output_size=(),
                          padding_algorithm="EXPLICIT", groups=1, dilations=(1, 1), data_format="NCHW"):
    return _wrap(TF.conv_transpose2d(_t(x), _t(filter), _t(bias), list(strides), list(paddings)[:2],
                                     list(output_padding) or 0, groups, list(dilations)))


def shuffle_channel(x, group=1):
    t = _t(x)
    n, c, h, w = t.shape
    return _wrap(t.view(n, group, c // group, h, w).transpose(1, 2).reshape(n, c, h, w))


def affine_channel(x, scale, bias, data_layout="NCHW"):
    t = _t(x)
    shape = (1, -1) + (1,) * (t.dim() - 2) if data_layout == "NCHW" else (1,) * (t.dim() - 1) + (-1,)
    return _wrap(t * _t(scale).view(shape) + _t(bias).view(shape))


# ------------------------------------------------------------------------------------------------ norms, losses, reductions
def p_norm(x, porder=2.0, axis=-1, epsilon=1e-12, keepdim=False, asvector=False):
    t = _t(x)
    if asvector:
        return _wrap(torch.linalg.vector_norm(t.reshape(-1), ord=porder, keepdim=keepdim))
    return _wrap(torch.linalg.vector_norm(t, ord=porder, dim=axis, keepdim=keepdim))


def frobenius_norm(x, axis=(), keep_dim=False, reduce_all=False):
    t = _t(x)
    dims = None if (reduce_all or not axis) else list(axis)
    return _wrap(torch.linalg.vector_norm(t, ord=2, dim=dims, keepdim=keep_dim))


def l1_norm(x):
    return _wrap(_t(x).abs().sum())


def mean_all(x):
    return _wrap(_t(x).mean())


def huber_loss(input, label, delta=1.0):
    r = _t(label) - _t(input)
    a = r.abs()
    return _wrap(torch.where(a <= delta, 0.5 * r * r, delta * (a - 0.5 * delta))), _wrap(r)


def hinge_loss(logits, labels):
    return _wrap(torch.clamp(1 - _t(logits) * (2 * _t(labels) - 1), min=0))


def matrix_rank_tol(x, atol_tensor, use_default_tol=True, hermitian=False):
    return _wrap(torch.linalg.matrix_rank(_t(x), tol=None if use_default_tol else _t(atol_tensor), hermitian=hermitian))


def matrix_rank_atol_rtol(x, atol, rtol=None, hermitian=False):
    return _wrap(torch.linalg.matrix_rank(_t(x), atol=_t(atol), rtol=_t(rtol) if rtol is not None else None,
                                          hermitian=hermitian))


# ------------------------------------------------------------------------------------------------ fills, random, views, copies
def fill(x, value=0.0):
    _t(x).fill_(float(value) if not isinstance(value, torch.Tensor) else float(_t(value).reshape(-1)[0]))
    return x


def full_int_array(value, dtype=torch.int64, place=None):
    return _wrap(torch.tensor(list(value), dtype=dtype if isinstance(dtype, torch.dtype) else torch.int64))


def full_with_tensor(value, shape, dtype=None):
    shp = [int(v) for v in (_t(shape).reshape(-1).tolist() if isinstance(shape, torch.Tensor) else shape)]
    v = _t(value)
    return _wrap(torch.full(shp, float(v.reshape(-1)[0]), dtype=dtype if isinstance(dtype, torch.dtype) else v.dtype,
                            device=v.device))


def full_batch_size_like(input, shape, dtype, value, input_dim_idx=0, output_dim_idx=0, place=None):
    shp = list(shape)
    shp[output_dim_idx] = _t(input).shape[input_dim_idx]
    return _wrap(torch.full(shp, float(value), dtype=dtype if isinstance(dtype, torch.dtype) else torch.float32,
                            device=_t(input).device))


def gaussian(shape, mean=0.0, std=1.0, seed=0, dtype=torch.float32, place=None):
    g = torch.Generator().manual_seed(seed) if seed else None
    return _wrap(torch.empty([int(s) for s in shape], dtype=dtype if isinstance(dtype, torch.dtype) else torch.float32)
                 .normal_(mean, std, generator=g))


def gaussian_inplace(x, mean=0.0, std=1.0, seed=0):
    _t(x).normal_(mean, std)
    return x


def uniform_inplace(x, min=-1.0, max=1.0, seed=0, diag_num=0, diag_step=0, diag_val=1.0):
    _t(x).uniform_(min, max)
    return x


def exponential_(x, lam=1.0):
    _t(x).exponential_(lam)
    return x


def truncated_gaussian_random(shape, mean=0.0, std=1.0, seed=0, a=-2.0, b=2.0, dtype=torch.float32, place=None):
    t = torch.empty([int(s) for s in shape], dtype=dtype if isinstance(dtype, torch.dtype) else torch.float32)
    torch.nn.init.trunc_normal_(t, mean, std, mean + a * std, mean + b * std)
    return _wrap(t)


def uniform_random_batch_size_like(input, shape, input_dim_idx=0, output_dim_idx=0, min=-1.0, max=1.0, seed=0, diag_num=0,
                                   diag_step=0, diag_val=1.0, dtype=torch.float32):
    shp = list(shape)
    shp[output_dim_idx] = _t(input).shape[input_dim_idx]
    return _wrap(torch.empty(shp, dtype=dtype if isinstance(dtype, torch.dtype) else torch.float32,
                             device=_t(input).device).uniform_(min, max))


def view_dtype(input, dtype):
    return _wrap(_t(input).view(dtype))


def view_shape(input, dims=()):
    return _wrap(_t(input).view(*[int(d) for d in dims]))


def view_slice(input, begin_idx, end_idx):
    return _wrap(_t(input)[int(begin_idx):int(end_idx)])


def split_with_num(x, num, axis=0):
    return _wrap(list(torch.chunk(_t(x), int(num), dim=int(axis if not isinstance(axis, torch.Tensor) else _t(axis)))))


def shape64(input):
    return _wrap(torch.tensor(list(_t(input).shape), dtype=torch.int64))


def share_data(x):
    return _wrap(_t(x).detach())


def assign_out_(x, output):
    _t(output).copy_(_t(x))
    return output


def assign_value_(output, shape, dtype, values, place=None):
    _t(output).copy_(torch.tensor(list(values), dtype=_t(output).dtype).reshape([int(s) for s in shape]))
    return output


def copy_to(x, place, blocking=True):
    dev = "cuda" if "gpu" in str(place).lower() or "cuda" in str(place).lower() else "cpu"
    return _wrap(_t(x).to(dev, non_blocking=not blocking))


def memcpy_d2h(x, dst_place_type=0):
    return _wrap(_t(x).to("cpu"))


def memcpy_h2d(x, dst_place_type=1):
    return _wrap(_t(x).to("cuda"))


def sync_calc_stream(x):
    if torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()
    return x


def depend(x, dep):
    return x


def trans_layout(x, perm):
    return _wrap(_t(x).permute(*[int(p) for p in perm]).contiguous())


def index_select_strided(x, index, axis=0):
    return _wrap(_t(x).select(int(axis), int(index)))


def repeat_interleave_with_tensor_index(x, repeats, axis=0, output_size=-1):
    return _wrap(torch.repeat_interleave(_t(x), _t(repeats), dim=int(axis)))


def set_value_with_tensor(x, values, starts, ends, steps, axes, decrease_axes=(), none_axes=()):
    t = _t(x).clone()
    idx = [slice(None)] * t.dim()
    for a, s, e, st in zip(axes, starts, ends, steps):
        idx[int(a)] = slice(int(s), int(e), int(st))
    t[tuple(idx)] = _t(values)
    return _wrap(t)


def fft_c2c(x, axes, normalization="backward", forward=True):
    f = torch.fft.fftn if forward else torch.fft.ifftn
    return _wrap(f(_t(x), dim=[int(a) for a in axes], norm=normalization))


def fft_r2c(x, axes, normalization="backward", forward=True, onesided=True):
    t = _t(x)
    if onesided:
        return _wrap(torch.fft.rfftn(t, dim=[int(a) for a in axes], norm=normalization))
    return _wrap(torch.fft.fftn(t.to(torch.complex64 if t.dtype == torch.float32 else torch.complex128),
                                dim=[int(a) for a in axes], norm=normalization))


def fft_c2r(x, axes, normalization="backward", forward=False, last_dim_size=0):
    s = None
    if last_dim_size:
        t = _t(x)
        s = [t.shape[int(a)] for a in axes]
        s[-1] = int(last_dim_size)
    return _wrap(torch.fft.irfftn(_t(x), s=s, dim=[int(a) for a in axes], norm=normalization))


def fused_elementwise(kind):
    f = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div}[kind]

    def op(x, y, axis=-1, *a, **k):
        return _wrap(f(_t(x), _t(y)))
    return op


fused_elementwise_add, fused_elementwise_sub = fused_elementwise("add"), fused_elementwise("sub")
fused_elementwise_mul, fused_elementwise_div = fused_elementwise("mul"), fused_elementwise("div")


def enable_check_model_nan_inf(x, flag=1):
    from .framework import flags as _f
    _f.set_flags({"FLAGS_check_nan_inf": bool(flag)})
    return x


def disable_check_model_nan_inf(x, flag=0):
    from .framework import flags as _f
    _f.set_flags({"FLAGS_check_nan_inf": bool(flag)})
    return x


def fill_diagonal(x, value=0.0, offset=0, wrap=False):
    t = _t(x)
    torch.diagonal(t, offset=int(offset)).fill_(float(value))
    return x


def fill_diagonal_tensor(x, y, offset=0, dim1=0, dim2=1):
    t = _t(x).clone()
    torch.diagonal(t, offset=int(offset), dim1=int(dim1), dim2=int(dim2)).copy_(_t(y))
    return _wrap(t)


def frame(x, frame_length, hop_length, axis=-1):
    """axis -1: [..., frame_length, n]; axis 0: [n, frame_length, ...] (also for 1-D input)."""
    t = _t(x)
    if axis != 0 and axis in (-1, t.dim() - 1):
        return _wrap(t.unfold(-1, int(frame_length), int(hop_length)).transpose(-1, -2))
    return _wrap(t.unfold(0, int(frame_length), int(hop_length)).movedim(-1, 1))


def overlap_add(x, hop_length, axis=-1):
    """Inverse layout of ``frame``: axis -1 takes [..., frame_length, n], axis 0 takes [n, frame_length, ...]."""
    t = _t(x)
    last = axis != 0 and axis in (-1, t.dim() - 1)
    if not last:
        t = t.movedim(0, -1).movedim(0, -1)            # [n, frame_length, ...] -> [..., frame_length, n]
    fl, n = t.shape[-2], t.shape[-1]
    out = torch.zeros(*t.shape[:-2], (n - 1) * int(hop_length) + fl, dtype=t.dtype, device=t.device)
    for i in range(n):
        out[..., i * int(hop_length):i * int(hop_length) + fl] += t[..., i]
    return _wrap(out if last else out.movedim(-1, 0))


def merged_adam_(param, grad, learning_rate, moment1, moment2, moment2_max, beta1_pow, beta2_pow, master_param=None,
                 beta1=0.9, beta2=0.999, epsilon=1e-8, multi_precision=False, use_global_beta_pow=False, amsgrad=False):
    for i in range(len(param)):
        adam_(param[i], grad[i], learning_rate[i] if isinstance(learning_rate, (list, tuple)) else learning_rate,
              moment1[i], moment2[i], None, beta1_pow[i], beta2_pow[i], master_param[i] if master_param else None, None,
              beta1, beta2, epsilon, False, 1000, multi_precision)
    return param, moment1, moment2, moment2_max, beta1_pow, beta2_pow, master_param


def merged_momentum_(param, grad, velocity, learning_rate, master_param=None, mu=0.9, use_nesterov=False,
                     regularization_method=(), regularization_coeff=(), multi_precision=False, rescale_grad=1.0):
    for i in range(len(param)):
        momentum_(param[i], grad[i], velocity[i], learning_rate[i] if isinstance(learning_rate, (list, tuple))
                  else learning_rate, master_param[i] if master_param else None, mu, use_nesterov,
                  regularization_method[i] if regularization_method else "",
                  regularization_coeff[i] if regularization_coeff else 0.0, multi_precision, rescale_grad)
    return param, velocity, master_param


def resolve(name):
    """Implementation of operator ``name`` from this table, or None."""
    import importlib
    g = globals()
    if name in g and callable(g[name]) and not name.startswith("_"):
        return g[name]
    if not name.startswith("_"):
        from . import _op_table_more, _op_table_seq
        for tier in (_op_table_more, _op_table_seq):
            fn = getattr(tier, name, None)
            if callable(fn) and getattr(fn, "__module__", "") == tier.__name__:
                return fn
    path = ALIASES.get(name)
    if path is not None:
        mod, _, attr = path.rpartition(".")
        try:
            return getattr(importlib.import_module(mod), attr)
        except (ImportError, AttributeError):
            return None
    if name in NOT_BUILT:
        reason = NOT_BUILT[name]

        def not_built(*a, **k):
            raise NotImplementedError(f"operator {name!r} belongs to a part that is not built: {reason}")
        not_built.__name__ = name
        not_built.not_built = reason
        return not_built
    return None
