"""Remaining ``paddle.nn.functional`` entries: in-place activations, pooling variants, additional losses, beam-search
helpers (python/paddle/nn/functional/{activation,pooling,loss,extension}.py)."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as TF

from ..._core.tensor import as_tensor


def _p(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else x


def _inplace(fn):
    def f(x, *a, **k):
        k.pop("name", None)
        r = fn(_p(x), *a, **k)
        with torch.no_grad():
            _p(x).copy_(r)
        return x
    return f


elu_ = _inplace(lambda x, alpha=1.0: TF.elu(x, alpha))
hardtanh_ = _inplace(lambda x, min=-1.0, max=1.0: TF.hardtanh(x, min, max))
leaky_relu_ = _inplace(lambda x, negative_slope=0.01: TF.leaky_relu(x, negative_slope))
softmax_ = _inplace(lambda x, axis=-1, dtype=None: torch.softmax(x, axis))
tanh_ = _inplace(torch.tanh)
thresholded_relu_ = _inplace(lambda x, threshold=1.0, value=0.0: torch.where(x > threshold, x, torch.full_like(x, value)))


def feature_alpha_dropout(x, p=0.5, training=True, name=None):
    return as_tensor(TF.feature_alpha_dropout(_p(x), p, training))


def lp_pool1d(x, norm_type, kernel_size, stride=None, padding=0, ceil_mode=False, data_format="NCL", name=None):
    return as_tensor(TF.lp_pool1d(_p(x), float(norm_type), kernel_size, stride, ceil_mode))


def lp_pool2d(x, norm_type, kernel_size, stride=None, padding=0, ceil_mode=False, data_format="NCHW", name=None):
    return as_tensor(TF.lp_pool2d(_p(x), float(norm_type), kernel_size, stride, ceil_mode))


def max_unpool1d(x, indices, kernel_size, stride=None, padding=0, data_format="NCL", output_size=None, name=None):
    return as_tensor(TF.max_unpool1d(_p(x), _p(indices).long(), kernel_size, stride, padding, output_size))


def max_unpool2d(x, indices, kernel_size, stride=None, padding=0, data_format="NCHW", output_size=None, name=None):
    return as_tensor(TF.max_unpool2d(_p(x), _p(indices).long(), kernel_size, stride, padding, output_size))


def max_unpool3d(x, indices, kernel_size, stride=None, padding=0, data_format="NCDHW", output_size=None, name=None):
    return as_tensor(TF.max_unpool3d(_p(x), _p(indices).long(), kernel_size, stride, padding, output_size))


def adaptive_max_pool3d(x, output_size, return_mask=False, name=None):
    out = TF.adaptive_max_pool3d(_p(x), output_size, return_indices=return_mask)
    return (as_tensor(out[0]), as_tensor(out[1])) if return_mask else as_tensor(out)


def fractional_max_pool2d(x, output_size, kernel_size=None, random_u=None, return_mask=False, name=None):
    ks = kernel_size or 2
    samples = None if random_u is None else torch.full((x.shape[0], x.shape[1], 2), float(random_u))
    out = TF.fractional_max_pool2d(_p(x), ks, output_size=output_size, return_indices=return_mask, _random_samples=samples)
    return (as_tensor(out[0]), as_tensor(out[1])) if return_mask else as_tensor(out)


def fractional_max_pool3d(x, output_size, kernel_size=None, random_u=None, return_mask=False, name=None):
    ks = kernel_size or 2
    samples = None if random_u is None else torch.full((x.shape[0], x.shape[1], 3), float(random_u))
    out = TF.fractional_max_pool3d(_p(x), ks, output_size=output_size, return_indices=return_mask, _random_samples=samples)
    return (as_tensor(out[0]), as_tensor(out[1])) if return_mask else as_tensor(out)


def _reduce(loss, reduction):
    if reduction == "mean":
        return as_tensor(loss.mean())
    if reduction == "sum":
        return as_tensor(loss.sum())
    return as_tensor(loss)


def dice_loss(input, label, epsilon=1e-5, name=None):
    x, y = _p(input), _p(label)
    onehot = TF.one_hot(y.squeeze(-1).long(), x.shape[-1]).to(x.dtype)
    dims = tuple(range(1, x.dim()))
    inter = (x * onehot).sum(dims)
    denom = x.sum(dims) + onehot.sum(dims)
    return as_tensor((1 - 2 * inter / (denom + epsilon)).mean())


def poisson_nll_loss(input, label, log_input=True, full=False, epsilon=1e-8, reduction="mean", name=None):
    return as_tensor(TF.poisson_nll_loss(_p(input), _p(label), log_input, full, eps=epsilon, reduction=reduction))


def multi_label_soft_margin_loss(input, label, weight=None, reduction="mean", name=None):
    return as_tensor(TF.multilabel_soft_margin_loss(_p(input), _p(label).to(input.dtype), _p(weight), reduction=reduction))


def multi_margin_loss(input, label, p=1, margin=1.0, weight=None, reduction="mean", name=None):
    return as_tensor(TF.multi_margin_loss(_p(input), _p(label).long(), p, margin, _p(weight), reduction=reduction))


def soft_margin_loss(input, label, reduction="mean", name=None):
    return as_tensor(TF.soft_margin_loss(_p(input), _p(label).to(input.dtype), reduction=reduction))


def gaussian_nll_loss(input, label, variance, full=False, epsilon=1e-6, reduction="mean", name=None):
    return as_tensor(TF.gaussian_nll_loss(_p(input), _p(label), _p(variance), full, epsilon, reduction))


def triplet_margin_with_distance_loss(input, positive, negative, distance_function=None, margin=1.0, swap=False,
                                      reduction="mean", name=None):
    return as_tensor(TF.triplet_margin_with_distance_loss(_p(input), _p(positive), _p(negative),
                                                          distance_function=distance_function, margin=margin, swap=swap,
                                                          reduction=reduction))


def npair_loss(anchor, positive, labels, l2_reg=0.002):
    a, p_, y = _p(anchor), _p(positive), _p(labels).reshape(-1, 1).float()
    same = (y == y.t()).float()
    target = same / same.sum(1, keepdim=True)
    logits = a @ p_.t()
    ce = (-target * torch.log_softmax(logits, 1)).sum(1).mean()
    reg = l2_reg * ((a ** 2).sum(1).mean() + (p_ ** 2).sum(1).mean()) * 0.25
    return as_tensor(ce + reg)


def hsigmoid_loss(input, label, num_classes, weight, bias=None, path_table=None, path_code=None, is_sparse=False, name=None):
    """Hierarchical sigmoid over the default complete binary tree (custom trees through path_table / path_code)."""
    x, y, w = _p(input), _p(label).reshape(-1).long(), _p(weight)
    losses = []
    depth = int(math.ceil(math.log2(max(num_classes, 2))))
    for i in range(x.shape[0]):
        if path_table is not None:
            nodes = [int(n) for n in _p(path_table)[i].tolist() if n >= 0]
            codes = [float(c) for c in _p(path_code)[i].tolist()][:len(nodes)]
        else:
            code = int(y[i]) + num_classes
            nodes, codes = [], []
            while code > 1:
                nodes.append(code // 2 - 1)
                codes.append(float(code % 2))
                code //= 2
        keep = [j for j, nd_ in enumerate(nodes) if 0 <= nd_ < w.shape[0]]     # a label beyond num_classes walks off the tree
        nodes, codes = [nodes[j] for j in keep], [codes[j] for j in keep]
        n = torch.tensor(nodes, dtype=torch.long)
        logit = w[n] @ x[i] + (_p(bias).reshape(-1)[n] if bias is not None else 0)
        losses.append(TF.binary_cross_entropy_with_logits(logit, torch.tensor(codes, dtype=x.dtype), reduction="sum"))
    return as_tensor(torch.stack(losses).reshape(-1, 1))


def margin_cross_entropy(logits, label, margin1=1.0, margin2=0.5, margin3=0.0, scale=64.0, group=None,
                         return_softmax=False, reduction="mean"):
    """ArcFace-style margins: cos(m1 * theta + m2) - m3 on the target logit, then scaled softmax cross-entropy."""
    x, y = _p(logits).float(), _p(label).reshape(-1).long()
    theta = torch.acos(x.clamp(-1 + 1e-7, 1 - 1e-7))
    target = torch.cos(margin1 * theta + margin2) - margin3
    onehot = TF.one_hot(y, x.shape[1]).bool()
    z = torch.where(onehot, target, x) * scale
    loss = TF.cross_entropy(z, y, reduction="none").unsqueeze(-1)
    out = _reduce(loss, reduction)
    return (out, as_tensor(torch.softmax(z, 1))) if return_softmax else out


def rnnt_loss(input, label, input_lengths, label_lengths, blank=0, fastemit_lambda=0.001, reduction="mean", name=None):
    """RNN-T loss by the forward algorithm in log space (input: [B, T, U+1, V] un-normalised logits)."""
    lp = torch.log_softmax(_p(input) if _p(input).dtype == torch.float64 else _p(input).float(), -1)
    B = lp.shape[0]
    losses = []
    for b in range(B):
        T, U = int(input_lengths[b]), int(label_lengths[b])
        y = _p(label)[b, :U].long()
        alpha = torch.full((T, U + 1), float("-inf"))
        alpha[0, 0] = 0.0
        for t in range(T):
            for u in range(U + 1):
                if t == 0 and u == 0:
                    continue
                a = alpha[t - 1, u] + lp[b, t - 1, u, blank] if t > 0 else torch.tensor(float("-inf"))
                c = alpha[t, u - 1] + lp[b, t, u - 1, y[u - 1]] if u > 0 else torch.tensor(float("-inf"))
                alpha[t, u] = torch.logaddexp(a, c)
        losses.append(-(alpha[T - 1, U] + lp[b, T - 1, U, blank]))
    return _reduce(torch.stack(losses), reduction)


def gather_tree(ids, parents):
    """Back-trace beam-search parents: ids/parents [max_time, batch, beam] -> full sequences."""
    ids, parents = _p(ids), _p(parents).long()
    T = ids.shape[0]
    out = torch.empty_like(ids)
    out[T - 1] = ids[T - 1]
    beam = torch.arange(ids.shape[2]).expand(ids.shape[1], -1).clone()
    for t in range(T - 1, 0, -1):
        beam = parents[t].gather(1, beam)
        out[t - 1] = ids[t - 1].gather(1, beam)
    return as_tensor(out)


def class_center_sample(label, num_classes, num_samples, group=None):
    """Keep every positive class centre, fill up to ``num_samples`` with random negatives; returns (remapped_label,
    sampled_class_index)."""
    y = _p(label).reshape(-1).long()
    pos = torch.unique(y)
    if pos.numel() < num_samples:
        mask = torch.ones(num_classes, dtype=torch.bool)
        mask[pos] = False
        neg = torch.nonzero(mask).reshape(-1)
        neg = neg[torch.randperm(neg.numel())[:num_samples - pos.numel()]]
        sampled = torch.cat([pos, neg]).sort().values
    else:
        sampled = pos
    remap = torch.full((num_classes,), -1, dtype=torch.long)
    remap[sampled] = torch.arange(sampled.numel())
    return as_tensor(remap[y]), as_tensor(sampled)


def sparse_attention(query, key, value, sparse_csr_offset, sparse_csr_columns, key_padding_mask=None, attn_mask=None, name=None):
    """Attention restricted to the CSR pattern (offset / columns per batch and head)."""
    q, k, v = _p(query).float(), _p(key).float(), _p(value).float()
    B, H, S, D = q.shape
    scores = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(D)
    mask = torch.zeros(B, H, S, S, dtype=torch.bool)
    off, cols = _p(sparse_csr_offset).long(), _p(sparse_csr_columns).long()
    for b in range(B):
        for h in range(H):
            for r in range(S):
                mask[b, h, r, cols[b, h, off[b, h, r]:off[b, h, r + 1]]] = True
    scores = scores.masked_fill(~mask.to(scores.device), float("-inf"))
    if key_padding_mask is not None:
        scores = scores + _p(key_padding_mask).float()[:, None, None, :]
    if attn_mask is not None:
        scores = scores + _p(attn_mask).float()
    return as_tensor(torch.matmul(torch.nan_to_num(torch.softmax(scores, -1)), v).to(query.dtype))


def adaptive_log_softmax_with_loss(input, label, head_weight, tail_weights, cutoffs, head_bias=None, name=None):
    x, y = _p(input), _p(label).long()
    n_clusters = len(cutoffs) - 1 if cutoffs[-1] > cutoffs[0] else len(cutoffs)
    cut = [0] + list(cutoffs)
    head = TF.linear(x, _p(head_weight).t(), _p(head_bias))
    head_lp = torch.log_softmax(head, 1)
    out = torch.zeros(x.shape[0], dtype=x.dtype)
    short = cut[1]
    for i in range(len(cut) - 1):
        lo, hi = cut[i], cut[i + 1]
        sel = torch.nonzero((y >= lo) & (y < hi)).reshape(-1)
        if sel.numel() == 0:
            continue
        if i == 0:
            out[sel] = head_lp[sel].gather(1, y[sel, None]).squeeze(1)
        else:
            w1, w2 = tail_weights[i - 1]
            h = TF.linear(TF.linear(x[sel], _p(w1).t()), _p(w2).t())
            lp = torch.log_softmax(h, 1)
            out[sel] = head_lp[sel, short + i - 1] + lp.gather(1, (y[sel] - lo)[:, None]).squeeze(1)
    return as_tensor(out), as_tensor(-out.mean())


def flash_attn_qkvpacked(qkv, dropout=0.0, causal=False, return_softmax=False, fixed_seed_offset=None, rng_name="",
                         training=True, name=None):
    """qkv: [batch, seq, 3 (or groups + 2), heads_k, head_dim] as in flash_attention.py:600."""
    from .flash_attention import flash_attention
    t = _p(qkv)
    g = t.shape[2] - 2
    q = t[:, :, :g].reshape(t.shape[0], t.shape[1], g * t.shape[3], t.shape[4])
    return flash_attention(as_tensor(q), as_tensor(t[:, :, g]), as_tensor(t[:, :, g + 1]), dropout, causal, return_softmax,
                           training=training)


def flash_attn_varlen_qkvpacked(qkv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale, dropout=0.0,
                                causal=False, return_softmax=False, fixed_seed_offset=None, rng_name="", varlen_padded=True,
                                training=True, name=None):
    """Packed variable-length form: sequences are processed one by one on the dense kernel."""
    from .flash_attention import flash_attention
    t = _p(qkv)
    cu = _p(cu_seqlens_q).tolist()
    outs = []
    g = t.shape[1] - 2
    for a, b in zip(cu[:-1], cu[1:]):
        seg = t[a:b]
        q = seg[:, :g].reshape(1, b - a, g * seg.shape[2], seg.shape[3])
        o, _ = flash_attention(as_tensor(q), as_tensor(seg[None, :, g]), as_tensor(seg[None, :, g + 1]), dropout, causal,
                               False, training=training)
        outs.append(_p(o)[0])
    return as_tensor(torch.cat(outs, 0)), None


def edit_distance(input, label, normalized=True, ignored_tokens=None, input_length=None, label_length=None):
    """Levenshtein distance between rows of two padded id matrices (python/paddle/nn/functional/loss.py ``edit_distance``):
    ``ignored_tokens`` are dropped from both first; ``normalized`` divides by the label length.
    -> (number of sequences [1] int64, distances [batch, 1] float32): the operator's output order, which is what the
    reference returns in dynamic mode."""
    a, b = _p(input).long(), _p(label).long()
    la = _p(input_length).reshape(-1).tolist() if input_length is not None else [a.shape[1]] * a.shape[0]
    lb = _p(label_length).reshape(-1).tolist() if label_length is not None else [b.shape[1]] * b.shape[0]
    drop = set(int(t) for t in (ignored_tokens or []))
    out = []
    for i in range(a.shape[0]):
        h = [t for t in a[i, :int(la[i])].tolist() if t not in drop]
        r = [t for t in b[i, :int(lb[i])].tolist() if t not in drop]
        prev = list(range(len(r) + 1))
        for x in range(1, len(h) + 1):
            cur = [x] + [0] * len(r)
            for y in range(1, len(r) + 1):
                cur[y] = min(prev[y] + 1, cur[y - 1] + 1, prev[y - 1] + (h[x - 1] != r[y - 1]))
            prev = cur
        d = float(prev[len(r)])
        out.append(d / max(len(r), 1) if normalized else d)
    return as_tensor(torch.tensor([a.shape[0]], dtype=torch.int64)), as_tensor(torch.tensor(out, dtype=torch.float32).reshape(-1, 1))
