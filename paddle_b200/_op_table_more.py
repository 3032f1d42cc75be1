"""More kernel-level operators behind ``paddle._C_ops`` (same contract as ``_op_table.py``): the fake-quantisation
family of quantisation-aware training, the remaining optimizer updates, recurrent cells, and assorted helpers.
References are the kernels under paddle/phi/kernels (``fake_quantize_kernel.*``, ``asgd_kernel``, ``nadam_kernel``,
``radam_kernel``, ``rprop_kernel``, ``ftrl_kernel``, ``decayed_adagrad_kernel``, ``edit_distance_kernel``,
``box_clip_kernel``, ``add_position_encoding_kernel``, ``gru_unit_kernel`` ...); formulas follow their documentation in
python/paddle/optimizer/*.py and python/paddle/nn/quant/*."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as TF

from ._op_table import _t, _wrap


# ------------------------------------------------------------------------------------------------ fake quantisation
def _qrange(bit_length):
    return float((1 << (int(bit_length) - 1)) - 1)


def _round(x, round_type):
    # 0: round half to even (rint), 1: round half away from zero
    return torch.round(x) if round_type == 0 else torch.sign(x) * torch.floor(torch.abs(x) + 0.5)


def fake_quantize_abs_max(x, bit_length=8, round_type=1):
    """-> (quantised values as floats in [-bnt, bnt], scale = max |x|)."""
    t = _t(x)
    scale = t.abs().max().reshape(1)
    bnt = _qrange(bit_length)
    q = _round(t / scale.clamp_min(1e-30) * bnt, round_type).clamp(-bnt, bnt)
    return _wrap(q), _wrap(scale)


def fake_quantize_dequantize_abs_max(x, bit_length=8, round_type=1):
    t = _t(x)
    q, scale = fake_quantize_abs_max(t, bit_length, round_type)
    return _wrap(_t(q) * _t(scale) / _qrange(bit_length)), scale


def fake_channel_wise_quantize_abs_max(x, bit_length=8, round_type=1, quant_axis=0, is_test=False):
    t = _t(x)
    dims = [d for d in range(t.dim()) if d != quant_axis]
    scale = t.abs().amax(dims, keepdim=True)
    bnt = _qrange(bit_length)
    q = _round(t / scale.clamp_min(1e-30) * bnt, round_type).clamp(-bnt, bnt)
    return _wrap(q), _wrap(scale.reshape(-1))


def fake_channel_wise_quantize_dequantize_abs_max(x, bit_length=8, round_type=1, quant_axis=0):
    t = _t(x)
    q, scale = fake_channel_wise_quantize_abs_max(t, bit_length, round_type, quant_axis)
    shape = [1] * t.dim()
    shape[quant_axis] = -1
    return _wrap(_t(q) * _t(scale).reshape(shape) / _qrange(bit_length)), scale


def fake_dequantize_max_abs(x, scale, max_range):
    return _wrap(_t(x) * _t(scale) / float(max_range))


def fake_channel_wise_dequantize_max_abs(x, scales, quant_bits=(8,), quant_axis=0, x_num_col_dims=1):
    t = _t(x).float()
    s0 = _t(scales[0])
    shape = [1] * t.dim()
    shape[quant_axis] = -1
    out = t * s0.reshape(shape) / _qrange(quant_bits[0])
    if len(scales) > 1 and scales[1] is not None:
        out = out * _t(scales[1]) / _qrange(quant_bits[1])
    return _wrap(out)


def fake_quantize_range_abs_max(x, in_scale, iter, window_size=10000, bit_length=8, is_test=False, round_type=1):
    """Scale = max of the current |x| and the running scale (the reference also keeps a window of past scales)."""
    t = _t(x)
    cur = t.abs().max().reshape(1)
    scale = _t(in_scale).reshape(1) if is_test else torch.maximum(cur, _t(in_scale).reshape(1))
    bnt = _qrange(bit_length)
    q = _round(t / scale.clamp_min(1e-30) * bnt, round_type).clamp(-bnt, bnt)
    return _wrap(q), _wrap(scale), _wrap(scale.clone())


def _moving_average_scale(t, in_scale, in_accum, in_state, moving_rate, is_test):
    if is_test:
        return _t(in_scale).reshape(1), in_state, in_accum
    cur = t.abs().max().reshape(1)
    state = (_t(in_state).reshape(1) if in_state is not None else torch.ones(1)) * moving_rate + 1.0
    accum = (_t(in_accum).reshape(1) if in_accum is not None else torch.zeros(1)) * moving_rate + cur
    return accum / state, state, accum


def fake_quantize_moving_average_abs_max(x, in_scale, in_accum=None, in_state=None, moving_rate=0.9, bit_length=8,
                                         is_test=False, round_type=1):
    t = _t(x)
    scale, state, accum = _moving_average_scale(t, in_scale, in_accum, in_state, moving_rate, is_test)
    bnt = _qrange(bit_length)
    q = _round(t / scale.clamp_min(1e-30) * bnt, round_type).clamp(-bnt, bnt)
    return _wrap(q), _wrap(scale), _wrap(state) if state is not None else None, _wrap(accum) if accum is not None else None


def fake_quantize_dequantize_moving_average_abs_max(x, in_scale, in_accum=None, in_state=None, moving_rate=0.9,
                                                    bit_length=8, is_test=False, round_type=1):
    q, scale, state, accum = fake_quantize_moving_average_abs_max(x, in_scale, in_accum, in_state, moving_rate, bit_length,
                                                                  is_test, round_type)
    return _wrap(_t(q) * _t(scale) / _qrange(bit_length)), scale, state, accum


def dequantize_abs_max(x, scale, max_range):
    return _wrap(_t(x).float() * _t(scale) / float(max_range))


def dequantize_log(x, dict):
    """int8 codes -> table values; negative codes mirror the table (dequantize_log_kernel)."""
    t = _t(x).to(torch.int64)
    table = _t(dict).float()
    return _wrap(torch.where(t < 0, -table[(t + 128).clamp(0, table.numel() - 1)], table[t.clamp(0, table.numel() - 1)]))


def apply_per_channel_scale(x, scales):
    return _wrap(_t(x) * _t(scales))


# ------------------------------------------------------------------------------------------------ optimizers
def asgd_(param, grad, learning_rate, d, y, n, master_param=None, multi_precision=False):
    """Averaged SGD (python/paddle/optimizer/asgd.py): d <- d - y + g, y <- g, param <- param - lr / n * d."""
    p = _t(master_param) if (multi_precision and master_param is not None) else _t(param)
    g = _t(grad).to(p.dtype)
    dd, yy = _t(d), _t(y)
    dd.copy_(dd - yy + g)
    yy.copy_(g)
    p.sub_(_t(learning_rate).to(p.dtype) / _t(n).to(p.dtype) * dd)
    if p is not _t(param):
        _t(param).copy_(p.to(_t(param).dtype))
    return param, d, y, master_param


def nadam_(param, grad, learning_rate, momentum_decay_pow, beta2_pow, mu_product, moment1, moment2, master_param=None,
           beta1=0.9, beta2=0.999, epsilon=1e-8, momentum_decay=0.004, multi_precision=False):
    """NAdam (python/paddle/optimizer/nadam.py)."""
    p = _t(master_param) if (multi_precision and master_param is not None) else _t(param)
    g = _t(grad).to(p.dtype)
    mdp, b2p, mup, m1, m2 = _t(momentum_decay_pow), _t(beta2_pow), _t(mu_product), _t(moment1), _t(moment2)
    step_decay = 0.96 ** momentum_decay                 # momentum_decay_pow holds 0.96 ^ (t * momentum_decay)
    mdp.mul_(step_decay)
    b2p.mul_(beta2)
    mu_t = beta1 * (1.0 - 0.5 * mdp)
    mu_t1 = beta1 * (1.0 - 0.5 * mdp * step_decay)
    mup.mul_(mu_t)
    m1.mul_(beta1).add_(g, alpha=1 - beta1)
    m2.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    lr = _t(learning_rate).to(p.dtype)
    m1_hat = mu_t1 * m1 / (1.0 - mup * mu_t1) + (1.0 - mu_t) * g / (1.0 - mup)
    m2_hat = m2 / (1.0 - b2p)
    p.sub_(lr * m1_hat / (m2_hat.sqrt() + epsilon))
    if p is not _t(param):
        _t(param).copy_(p.to(_t(param).dtype))
    return param, momentum_decay_pow, beta2_pow, mu_product, moment1, moment2, master_param


def radam_(param, grad, learning_rate, beta1_pow, beta2_pow, rho, moment1, moment2, master_param=None, beta1=0.9,
           beta2=0.999, epsilon=1e-8, multi_precision=False):
    """Rectified Adam (python/paddle/optimizer/radam.py)."""
    p = _t(master_param) if (multi_precision and master_param is not None) else _t(param)
    g = _t(grad).to(p.dtype)
    b1p, b2p, rh, m1, m2 = _t(beta1_pow), _t(beta2_pow), _t(rho), _t(moment1), _t(moment2)
    rho_inf = 2.0 / (1.0 - beta2) - 1.0
    b1p.mul_(beta1)
    b2p.mul_(beta2)
    m1.mul_(beta1).add_(g, alpha=1 - beta1)
    m2.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    # t from beta2^t: rho_t = rho_inf - 2 t beta2^t / (1 - beta2^t)
    t_step = torch.log(b2p) / math.log(beta2)
    rho_t = rho_inf - 2.0 * t_step * b2p / (1.0 - b2p)
    rh.copy_(rho_t.reshape(rh.shape))
    lr = _t(learning_rate).to(p.dtype)
    m1_hat = m1 / (1.0 - b1p)
    if float(rho_t) > 5.0:
        l_t = torch.sqrt(1.0 - b2p) / (m2.sqrt() + epsilon)
        r_t = math.sqrt(max(((float(rho_t) - 4) * (float(rho_t) - 2) * rho_inf) / ((rho_inf - 4) * (rho_inf - 2) * float(rho_t)), 0.0))
        p.sub_(lr * m1_hat * r_t * l_t)
    else:
        p.sub_(lr * m1_hat)
    if p is not _t(param):
        _t(param).copy_(p.to(_t(param).dtype))
    return param, beta1_pow, beta2_pow, rho, moment1, moment2, master_param


def rprop_(param, grad, prev, learning_rate, master_param=None, learning_rate_range=None, etas=None, multi_precision=False):
    """Resilient back-propagation (python/paddle/optimizer/rprop.py): per-element step sizes grow by eta+ while the
    gradient keeps its sign, shrink by eta- when it flips (and that element's gradient is dropped for the step)."""
    p = _t(master_param) if (multi_precision and master_param is not None) else _t(param)
    g = _t(grad).to(p.dtype).clone()
    pv, lr = _t(prev), _t(learning_rate)
    lo, hi = (float(v) for v in _t(learning_rate_range).reshape(-1)[:2]) if learning_rate_range is not None else (1e-5, 50.0)
    em, ep = (float(v) for v in _t(etas).reshape(-1)[:2]) if etas is not None else (0.5, 1.2)
    sign = g * pv
    factor = torch.where(sign > 0, torch.full_like(g, ep), torch.where(sign < 0, torch.full_like(g, em), torch.ones_like(g)))
    lr.copy_((lr * factor).clamp(lo, hi))
    g = torch.where(sign < 0, torch.zeros_like(g), g)
    p.sub_(torch.sign(g) * lr)
    pv.copy_(g)
    if p is not _t(param):
        _t(param).copy_(p.to(_t(param).dtype))
    return param, prev, learning_rate, master_param


def ftrl(param, squared_accumulator, linear_accumulator, grad, learning_rate, l1=0.0, l2=0.0, lr_power=-0.5):
    """Follow-the-regularised-leader (ftrl_kernel)."""
    p, sq, lin, g = _t(param), _t(squared_accumulator), _t(linear_accumulator), _t(grad)
    lr = float(_t(learning_rate).reshape(-1)[0])
    new_sq = sq + g * g
    if lr_power == -0.5:
        sigma = (new_sq.sqrt() - sq.sqrt()) / lr
    else:
        sigma = (new_sq.pow(-lr_power) - sq.pow(-lr_power)) / lr
    lin_new = lin + g - sigma * p
    quad = (new_sq.sqrt() if lr_power == -0.5 else new_sq.pow(-lr_power)) / lr + 2.0 * l2
    pre = torch.clamp(lin_new, -l1, l1) - lin_new
    p_new = torch.where(lin_new.abs() > l1, pre / quad, torch.zeros_like(p))
    return _wrap(p_new), _wrap(new_sq), _wrap(lin_new)


def decayed_adagrad(param, grad, moment, learning_rate, decay=0.95, epsilon=1e-6):
    p, g, m = _t(param), _t(grad), _t(moment)
    m_new = decay * m + (1.0 - decay) * g * g
    lr = float(_t(learning_rate).reshape(-1)[0])
    return _wrap(p - lr * g / (m_new.sqrt() + epsilon)), _wrap(m_new)


def average_accumulates_(param, in_sum_1, in_sum_2, in_sum_3, in_num_accumulates, in_old_num_accumulates,
                         in_num_updates, average_window=0.0, max_average_window=2 ** 63 - 1, min_average_window=10000):
    """Running sums of the parameter for ModelAverage (average_accumulates_kernel): sum_1 collects the current window,
    spills into sum_2 every 16384 updates, and a finished window moves everything into sum_3."""
    s1, s2, s3 = _t(in_sum_1), _t(in_sum_2), _t(in_sum_3)
    na, ona, nu = _t(in_num_accumulates), _t(in_old_num_accumulates), _t(in_num_updates)
    nu.add_(1)
    na.add_(1)
    s1.add_(_t(param).to(s1.dtype))
    if int(nu) % 16384 == 0:
        s2.add_(s1)
        s1.zero_()
    if int(na) >= min_average_window and int(na) >= min(max_average_window, int(nu) * average_window):
        s3.copy_(s1 + s2)
        s1.zero_()
        s2.zero_()
        ona.copy_(na)
        na.zero_()
    return in_sum_1, in_sum_2, in_sum_3, in_num_accumulates, in_old_num_accumulates, in_num_updates


# ------------------------------------------------------------------------------------------------ assorted
def edit_distance(hyps, refs, hypslength=None, refslength=None, normalized=False):
    """Levenshtein distance per row of two padded int matrices -> (sequence count [1] int64, distances [B, 1] fp32), the
    output order of the operator's definition."""
    h, r = _t(hyps), _t(refs)
    B = h.shape[0]
    hl = _t(hypslength).reshape(-1).tolist() if hypslength is not None else [h.shape[1]] * B
    rl = _t(refslength).reshape(-1).tolist() if refslength is not None else [r.shape[1]] * B
    out = torch.zeros(B, 1)
    for b in range(B):
        a, c = h[b, :int(hl[b])].tolist(), r[b, :int(rl[b])].tolist()
        prev = list(range(len(c) + 1))
        for i, x in enumerate(a, 1):
            cur = [i] + [0] * len(c)
            for j, y in enumerate(c, 1):
                cur[j] = min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (x != y))
            prev = cur
        d = float(prev[-1])
        out[b, 0] = d / max(len(c), 1) if normalized else d
    return _wrap(torch.tensor([B], dtype=torch.int64, device=h.device)), _wrap(out.to(h.device))


def box_clip(input, im_info):
    """Clip boxes [.., 4] to the image: im_info rows are (height, width, scale)."""
    b, info = _t(input), _t(im_info)
    h = (info[..., 0] / info[..., 2]).round() - 1
    w = (info[..., 1] / info[..., 2]).round() - 1
    shape = [-1] + [1] * (b.dim() - 2)
    out = b.clone()
    out[..., 0::2] = torch.minimum(torch.clamp_min(b[..., 0::2], 0), w.reshape(shape + [1]) if b.dim() > 2 else w.reshape(-1, 1))
    out[..., 1::2] = torch.minimum(torch.clamp_min(b[..., 1::2], 0), h.reshape(shape + [1]) if b.dim() > 2 else h.reshape(-1, 1))
    return _wrap(out)


def add_position_encoding(x, alpha=1.0, beta=1.0):
    """alpha * x + beta * sinusoidal position encoding over [batch, seq, dim] (first half sin, second half cos)."""
    t = _t(x)
    _, S, D = t.shape
    half = D // 2
    pos = torch.arange(S, dtype=torch.float32, device=t.device).unsqueeze(1)
    div = torch.pow(10000.0, torch.arange(half, dtype=torch.float32, device=t.device) / max(half - 1, 1))
    pe = torch.cat([torch.sin(pos / div), torch.cos(pos / div)], 1)
    if pe.shape[1] < D:
        pe = TF.pad(pe, (0, D - pe.shape[1]))
    return _wrap(alpha * t + beta * pe.to(t.dtype))


_UNARY = {"relu": torch.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh, "gelu": TF.gelu, "scale": None}
_BINARY = {"elementwise_add": torch.add, "elementwise_mul": torch.mul, "elementwise_sub": torch.sub}


def fused_elemwise_activation(x, y, functor_list, axis=-1, scale=0.0, save_intermediate_out=False):
    """``functor_list`` = [f, g]: unary(binary(x, y)) when f is the unary one, else binary(x, unary(y))
    (fused_elemwise_activation_kernel).  Returns (out, intermediate)."""
    a, b = _t(x), _t(y)
    f, g = functor_list

    def unary(name, v):
        return v * scale if name == "scale" else _UNARY[name](v)
    if f in _BINARY:
        inter = unary(g, b)
        return _wrap(_BINARY[f](a, inter)), _wrap(inter)
    inter = _BINARY[g](a, b)
    return _wrap(unary(f, inter)), _wrap(inter)


def fused_elemwise_add_activation(x, y, functor_list, axis=-1, scale=0.0, save_intermediate_out=False):
    return fused_elemwise_activation(x, y, functor_list, axis, scale, save_intermediate_out)


def fused_fc_elementwise_layernorm(x, w, y, bias0=None, scale=None, bias1=None, x_num_col_dims=1, activation_type="",
                                   epsilon=1e-5, begin_norm_axis=1):
    """layer_norm(act(x w + bias0) + y) (fused_fc_elementwise_layernorm_kernel) -> (out, mean, variance)."""
    a = _t(x)
    h = a.reshape(int(math.prod(a.shape[:x_num_col_dims])), -1) @ _t(w)
    if bias0 is not None:
        h = h + _t(bias0)
    if activation_type == "relu":
        h = torch.relu(h)
    h = h + _t(y).reshape(h.shape)
    mean = h.mean(-1, keepdim=True)
    var = h.var(-1, unbiased=False, keepdim=True)
    out = (h - mean) / torch.sqrt(var + epsilon)
    if scale is not None:
        out = out * _t(scale)
    if bias1 is not None:
        out = out + _t(bias1)
    return _wrap(out), _wrap(mean.reshape(-1)), _wrap(var.reshape(-1))


def add_group_norm_silu(x, residual=None, scale=None, bias=None, epsilon=1e-5, groups=-1, data_format="NCHW",
                        activation=""):
    """group_norm(x + residual) followed by silu when asked -> (out, residual_out, mean, variance)."""
    t = _t(x)
    if residual is not None:
        t = t + _t(residual)
    nchw = t if data_format == "NCHW" else t.movedim(-1, 1)
    g = groups if groups > 0 else nchw.shape[1]
    out = TF.group_norm(nchw, g, _t(scale) if scale is not None else None, _t(bias) if bias is not None else None, epsilon)
    if activation == "silu":
        out = TF.silu(out)
    flat = nchw.reshape(nchw.shape[0], g, -1).float()
    out = out if data_format == "NCHW" else out.movedim(1, -1)
    return _wrap(out), _wrap(t), _wrap(flat.mean(-1)), _wrap(flat.var(-1, unbiased=False))


def embedding_with_scaled_gradient(x, weight, padding_idx=-1):
    """Embedding lookup whose weight gradient is divided by the number of times each row was looked up."""
    ids, w = _t(x), _t(weight)
    counts = torch.bincount(ids.reshape(-1), minlength=w.shape[0]).clamp_min(1).to(w.dtype)
    scaled = w.detach() + (w - w.detach()) / counts.unsqueeze(1) * 1.0
    # forward value equals w; backward flows through the scaled term only
    out = TF.embedding(ids, w.detach() + (scaled - scaled.detach()), padding_idx=None if padding_idx < 0 else padding_idx)
    return _wrap(out)


def coalesce_tensor(input, dtype=None, copy_data=False, set_constant=False, persist_output=False, constant=0.0,
                    use_align=True, align_size=-1, size_of_dtype=-1, concated_shapes=(), concated_ranks=()):
    """Lay the tensors of ``input`` out in ONE flat buffer (256-byte aligned slots) and return views into it plus the
    buffer (coalesce_tensor_kernel: the fused-buffer primitive of gradient fusion)."""
    ts = [_t(t) for t in input]
    dt = ts[0].dtype
    align = max(1, 256 // ts[0].element_size()) if use_align else 1
    offs, total = [], 0
    for t in ts:
        offs.append(total)
        total += (t.numel() + align - 1) // align * align
    flat = torch.full((total,), float(constant), dtype=dt, device=ts[0].device) if set_constant \
        else torch.zeros(total, dtype=dt, device=ts[0].device)
    outs = []
    for t, o in zip(ts, offs):
        v = flat[o:o + t.numel()].view(t.shape)
        if copy_data and not set_constant:
            v.copy_(t)
        outs.append(_wrap(v))
    return outs, _wrap(flat)


def partial_allgather(x, nranks, rank, ring_id=0, group=None):
    """Every rank contributes slice ``rank`` of its flattened tensor; the result is the concatenation
    (partial_allgather_kernel; used by pipeline p2p to avoid sending tensor-parallel duplicates)."""
    from .distributed import collective as C
    t = _t(x).contiguous()
    flat = t.reshape(-1)
    per = flat.numel() // nranks
    if nranks == 1 or not C.is_initialized():
        return x
    out = torch.empty_like(flat)
    C.all_gather_into_tensor(out, flat[rank * per:(rank + 1) * per].contiguous(), group=group)
    return _wrap(out.view(t.shape))


def sync_batch_norm_(x, mean, variance, scale, bias, is_test=False, momentum=0.9, epsilon=1e-5, data_format="NCHW",
                     use_global_stats=False, trainable_statistics=False, group=None):
    """Batch norm whose batch statistics are averaged over the data-parallel group
    (sync_batch_norm_kernel) -> (out, mean_out, variance_out, saved_mean, saved_inv_std, reserve)."""
    from .distributed import collective as C
    t = _t(x)
    nchw = t if data_format == "NCHW" else t.movedim(-1, 1)
    dims = [0] + list(range(2, nchw.dim()))
    rm, rv = _t(mean), _t(variance)
    if is_test or use_global_stats:
        bm, bv = rm, rv
    else:
        n = torch.tensor([float(nchw.numel() // nchw.shape[1])], device=t.device)
        s1, s2 = nchw.float().sum(dims), (nchw.float() ** 2).sum(dims)
        if C.is_initialized() and C.get_world_size() > 1:
            packed = torch.cat([s1, s2, n])
            C.all_reduce(packed, group=group)
            s1, s2, n = packed[:s1.numel()], packed[s1.numel():-1], packed[-1:]
        bm = s1 / n
        bv = s2 / n - bm * bm
        rm.mul_(momentum).add_(bm.to(rm.dtype), alpha=1 - momentum)
        rv.mul_(momentum).add_(bv.to(rv.dtype), alpha=1 - momentum)
    shape = [1, -1] + [1] * (nchw.dim() - 2)
    inv = torch.rsqrt(bv.float() + epsilon)
    out = (nchw.float() - bm.float().reshape(shape)) * inv.reshape(shape)
    if scale is not None:
        out = out * _t(scale).float().reshape(shape)
    if bias is not None:
        out = out + _t(bias).float().reshape(shape)
    out = out.to(t.dtype)
    out = out if data_format == "NCHW" else out.movedim(1, -1)
    return _wrap(out), mean, variance, _wrap(bm), _wrap(inv), None


def merge_selected_rows(x):
    """Rows with the same index are summed.  ``x`` = (rows int64 [n], values [n, ...]) -> (unique rows, summed values)."""
    rows, vals = _t(x[0]), _t(x[1])
    uniq, inv = torch.unique(rows, return_inverse=True)
    out = torch.zeros((uniq.numel(), *vals.shape[1:]), dtype=vals.dtype, device=vals.device)
    out.index_add_(0, inv, vals)
    return _wrap(uniq), _wrap(out)


def set(x, source, dims=(), stride=(), offset=0):
    """``x`` becomes a view of ``source``'s storage with the given sizes / strides / offset (set_kernel)."""
    s = _t(source)
    sizes = list(dims) if len(dims) else list(s.shape)
    strides = list(stride) if len(stride) else list(torch.empty(sizes).stride())
    _t(x).set_(s.untyped_storage(), int(offset), sizes, strides)
    return x


def data(name, shape, dtype="float32", place=None):
    from . import static
    return static.data(name, shape, dtype)


def accuracy_check(x, y, fn_name="", rtol=None, atol=None, equal_nan=False):
    """Raises when ``x`` and ``y`` differ beyond the tolerances; returns a boolean tensor otherwise.  Tolerances left
    unset come from ``FLAGS_accuracy_check_{atol,rtol}_{fp32,fp16,bf16}`` by the dtype of ``x``."""
    if rtol is None or atol is None:
        from .framework.flags import flag
        kind = {torch.float16: "fp16", torch.bfloat16: "bf16"}.get(_t(x).dtype, "fp32")
        rtol = flag(f"accuracy_check_rtol_{kind}") if rtol is None else rtol
        atol = flag(f"accuracy_check_atol_{kind}") if atol is None else atol
    ok = torch.allclose(_t(x).float(), _t(y).float(), rtol=rtol, atol=atol, equal_nan=equal_nan)
    if not ok:
        diff = (_t(x).float() - _t(y).float()).abs().max().item()
        raise AssertionError(f"accuracy check failed for {fn_name or 'tensor'}: max |x - y| = {diff}")
    return _wrap(torch.tensor([True]))


def gru_unit(input, hidden_prev, weight, bias=None, activation=2, gate_activation=1, origin_mode=False):
    """One GRU step (gru_unit_kernel): ``input`` [B, 3D] holds the projected update / reset / candidate inputs,
    ``weight`` [D, 3D] the hidden-to-hidden matrices ([:, :2D] gates, [:, 2D:] candidate).  Activations: 0 identity,
    1 sigmoid, 2 tanh, 3 relu.  -> (gate, reset_hidden_prev, hidden)."""
    acts = {0: lambda v: v, 1: torch.sigmoid, 2: torch.tanh, 3: torch.relu}
    x, h, w = _t(input), _t(hidden_prev), _t(weight)
    D = h.shape[1]
    if bias is not None:
        x = x + _t(bias).reshape(1, -1)
    g = x[:, :2 * D] + h @ w[:, :2 * D]
    u, r = acts[gate_activation](g[:, :D]), acts[gate_activation](g[:, D:])
    rh = r * h
    c = acts[activation](x[:, 2 * D:] + rh @ w[:, 2 * D:])
    new_h = (u * h + (1 - u) * c) if origin_mode else ((1 - u) * h + u * c)
    return _wrap(torch.cat([u, r, c], 1)), _wrap(rh), _wrap(new_h)


def bipartite_match(dist_mat, match_type="bipartite", dist_threshold=0.5):
    """Greedy bipartite matching of columns to rows by descending distance (bipartite_match_kernel) ->
    (col_to_row_match_indices [1, cols] int32, col_to_row_match_dist [1, cols])."""
    d = _t(dist_mat).clone().float()
    rows, cols = d.shape
    idx = torch.full((1, cols), -1, dtype=torch.int32)
    dist = torch.zeros(1, cols)
    work = d.clone()
    for _ in range(min(rows, cols)):
        flat = int(torch.argmax(work))
        r, c = divmod(flat, cols)
        if work[r, c] <= 0:
            break
        idx[0, c], dist[0, c] = r, d[r, c]
        work[r, :] = -1
        work[:, c] = -1
    if match_type == "per_prediction":
        best, arg = torch.max(d, 0)
        extra = (idx[0] < 0) & (best >= dist_threshold)
        idx[0, extra] = arg[extra].to(torch.int32)
        dist[0, extra] = best[extra]
    return _wrap(idx.to(d.device)), _wrap(dist.to(d.device))
