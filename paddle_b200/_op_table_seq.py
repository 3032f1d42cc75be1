"""Recurrent and detection operators behind ``paddle._C_ops`` (same contract as ``_op_table.py``).

``rnn`` is the operator ``paddle.nn.SimpleRNN / LSTM / GRU`` lower to (paddle/phi/kernels/gpu/rnn_kernel.cu.cc,
python/paddle/nn/layer/rnn.py:1480-1640): multi-layer, optionally bidirectional, time-major input, per-sequence
lengths.  Without lengths the cuDNN sequence kernels are used through torch; with lengths the recurrence is stepped
here so that padded steps neither change the state nor produce output.  ``cudnn_lstm``, ``lstm`` and ``gru`` are the
older forms (paddle/phi/kernels/gpu/cudnn_lstm_kernel.cu, paddle/phi/kernels/impl/lstm_kernel_impl.h,
gru_kernel_impl.h).  Detection: ``multiclass_nms3`` (paddle/phi/kernels/cpu/multiclass_nms3_kernel.cc),
``yolo_box_head`` / ``yolo_box_post`` (paddle/phi/kernels/gpu/yolo_box_head_kernel.cu, yolo_box_post_kernel.cu),
``collect_fpn_proposals`` (paddle/phi/kernels/gpu/collect_fpn_proposals_kernel.cu), ``correlation``
(paddle/phi/kernels/gpu/correlation_kernel.cu)."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as TF

from ._op_table import _t, _wrap

_GATES = {"LSTM": 4, "GRU": 3, "RNN_TANH": 1, "RNN_RELU": 1}


# --------------------------------------------------------------------------------------------------------- recurrent
def _split_weights(weight_list, num_layers, dirs):
    """Paddle's flat list holds every (w_ih, w_hh) pair first, then every (b_ih, b_hh) pair, layer-major and
    direction-minor.  -> per (layer, direction): (w_ih, w_hh, b_ih or None, b_hh or None)."""
    ws = [_t(w) for w in weight_list]
    n = num_layers * dirs
    has_bias = len(ws) >= 4 * n
    out = []
    for i in range(n):
        w_ih, w_hh = ws[2 * i], ws[2 * i + 1]
        b_ih, b_hh = (ws[2 * n + 2 * i], ws[2 * n + 2 * i + 1]) if has_bias else (None, None)
        out.append((w_ih, w_hh, b_ih, b_hh))
    return out, has_bias


def _cell(mode, x_proj, h, c, w_hh, b_hh):
    """One step from the already projected input ``x_proj`` = x W_ih^T + b_ih.  Gate order: LSTM i, f, g, o;
    GRU r, z, n (the cuDNN order, which Paddle's cells share)."""
    hp = h @ w_hh.t()
    if b_hh is not None:
        hp = hp + b_hh
    if mode == "LSTM":
        i, f, g, o = (x_proj + hp).chunk(4, -1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        return torch.sigmoid(o) * torch.tanh(c), c
    if mode == "GRU":
        xr, xz, xn = x_proj.chunk(3, -1)
        hr, hz, hn = hp.chunk(3, -1)
        r, z = torch.sigmoid(xr + hr), torch.sigmoid(xz + hz)
        n = torch.tanh(xn + r * hn)
        return (1 - z) * n + z * h, c
    act = torch.tanh if mode == "RNN_TANH" else torch.relu
    return act(x_proj + hp), c


def _run_direction(mode, x, h, c, weights, lengths, reverse):
    """x: [T, B, I] -> ([T, B, H], last h, last c).  With ``lengths`` a sequence's state freezes after its last valid
    step (in the reverse direction it starts at that step) and the outputs of its padded steps are zero."""
    w_ih, w_hh, b_ih, b_hh = weights
    T = x.shape[0]
    xp = x @ w_ih.t()
    if b_ih is not None:
        xp = xp + b_ih
    outs = [None] * T
    steps = range(T - 1, -1, -1) if reverse else range(T)
    for t in steps:
        nh, nc = _cell(mode, xp[t], h, c, w_hh, b_hh)
        if lengths is not None:
            live = (lengths > t).to(x.dtype).unsqueeze(-1)
            h = live * nh + (1 - live) * h
            if c is not None:
                c = live * nc + (1 - live) * c
            outs[t] = live * nh
        else:
            h, c = nh, nc
            outs[t] = nh
    return torch.stack(outs, 0), h, c


def rnn(x, pre_state, weight_list, sequence_length=None, dropout_state_in=None, dropout_prob=0.0, is_bidirec=False,
        input_size=10, hidden_size=100, num_layers=1, mode="RNN_TANH", seed=0, is_test=False):
    """-> (out [T, B, dirs * H], dropout_state_out, [h_n (, c_n)] each [num_layers * dirs, B, H], reserve)."""
    if mode not in _GATES:
        raise ValueError(f"rnn mode {mode!r}; expected one of {sorted(_GATES)}")
    xt = _t(x)
    dirs = 2 if is_bidirec else 1
    states = [_t(s) for s in (pre_state if isinstance(pre_state, (list, tuple)) else [pre_state])]
    h0 = states[0]
    c0 = states[1] if mode == "LSTM" else None
    per, has_bias = _split_weights(weight_list, num_layers, dirs)
    lengths = _t(sequence_length).to(xt.device) if sequence_length is not None else None
    train = (not is_test) and dropout_prob > 0
    if lengths is None:
        flat = []
        for w_ih, w_hh, b_ih, b_hh in per:
            flat += [w_ih, w_hh] + ([b_ih, b_hh] if has_bias else [])
        if seed and train:
            torch.manual_seed(seed)
        if mode == "LSTM":
            out, hn, cn = torch._VF.lstm(xt, (h0, c0), flat, has_bias, num_layers, float(dropout_prob), train, is_bidirec, False)
            final = [hn, cn]
        elif mode == "GRU":
            out, hn = torch._VF.gru(xt, h0, flat, has_bias, num_layers, float(dropout_prob), train, is_bidirec, False)
            final = [hn]
        else:
            fn = torch._VF.rnn_tanh if mode == "RNN_TANH" else torch._VF.rnn_relu
            out, hn = fn(xt, h0, flat, has_bias, num_layers, float(dropout_prob), train, is_bidirec, False)
            final = [hn]
    else:
        layer_in = xt
        hs, cs = [], []
        for layer in range(num_layers):
            outs = []
            for d in range(dirs):
                idx = layer * dirs + d
                o, h, c = _run_direction(mode, layer_in, h0[idx], c0[idx] if c0 is not None else None, per[idx], lengths, d == 1)
                outs.append(o)
                hs.append(h)
                cs.append(c)
            layer_in = torch.cat(outs, -1) if dirs == 2 else outs[0]
            if train and layer < num_layers - 1:
                layer_in = TF.dropout(layer_in, dropout_prob, True)
        out = layer_in
        final = [torch.stack(hs, 0)] + ([torch.stack(cs, 0)] if mode == "LSTM" else [])
    empty = torch.empty(0, dtype=torch.uint8, device=xt.device)
    return _wrap(out), _wrap(empty), [_wrap(s) for s in final], _wrap(empty.clone())


def cudnn_lstm(x, init_h, init_c, w=None, weight_list=None, sequence_length=None, dropout_prob=0.0, is_bidirec=False,
               hidden_size=100, num_layers=1, is_test=False, seed=0):
    """LSTM over time-major ``x``.  Weights come either as ``weight_list`` (the layout of ``rnn``) or as one flat
    buffer ``w`` holding, in the same order, every matrix and then every bias.
    -> (out, last_h, last_c, reserve, state_out)."""
    xt = _t(x)
    dirs = 2 if is_bidirec else 1
    if weight_list is None:
        flat = _t(w).reshape(-1)
        I, H = xt.shape[-1], hidden_size
        shapes = []
        for layer in range(num_layers):
            in_sz = I if layer == 0 else H * dirs
            for _ in range(dirs):
                shapes += [(4 * H, in_sz), (4 * H, H)]
        shapes += [(4 * H,)] * (2 * num_layers * dirs)
        weight_list, off = [], 0
        for s in shapes:
            n = math.prod(s)
            weight_list.append(flat[off:off + n].reshape(s))
            off += n
        if off != flat.numel():
            raise ValueError(f"flat LSTM weight has {flat.numel()} elements, the layout needs {off}")
    out, _, (hn, cn), reserve = rnn(x, [init_h, init_c], weight_list, sequence_length, None, dropout_prob, is_bidirec,
                                    xt.shape[-1], hidden_size, num_layers, "LSTM", seed, is_test)
    return out, hn, cn, reserve, _wrap(torch.empty(0, dtype=torch.uint8, device=xt.device))


_ACT = {"sigmoid": torch.sigmoid, "tanh": torch.tanh, "relu": torch.relu, "identity": lambda v: v}


def _as_batch(t):
    """[T, D] (one sequence) or [B, T, D] -> ([B, T, D], was 2-D)."""
    return (t.unsqueeze(0), True) if t.dim() == 2 else (t, False)


def gru(input, h0=None, weight=None, bias=None, activation="tanh", gate_activation="sigmoid", is_reverse=False,
        origin_mode=False, is_test=False):
    """The older GRU operator: ``input`` holds x W_x already ([T, 3D] for one sequence or [B, T, 3D]; columns update |
    reset | candidate), ``weight`` [D, 3D] = [W_uh W_rh | W_ch].  -> (batch_gate, batch_reset_hidden_prev,
    batch_hidden, hidden), all in the layout of ``input``."""
    xin, squeeze = _as_batch(_t(input))
    w = _t(weight)
    D = w.shape[0]
    if bias is not None:
        xin = xin + _t(bias).reshape(1, 1, -1)
    B, T, _ = xin.shape
    h = _t(h0).reshape(B, D) if h0 is not None else xin.new_zeros(B, D)
    ga, ca = _ACT[gate_activation], _ACT[activation]
    gates, resets, hiddens = [None] * T, [None] * T, [None] * T
    for t in (range(T - 1, -1, -1) if is_reverse else range(T)):
        xt = xin[:, t]
        g = xt[:, :2 * D] + h @ w[:, :2 * D]
        u, r = ga(g[:, :D]), ga(g[:, D:])
        rh = r * h
        c = ca(xt[:, 2 * D:] + rh @ w[:, 2 * D:])
        h = (u * h + (1 - u) * c) if origin_mode else ((1 - u) * h + u * c)
        gates[t], resets[t], hiddens[t] = torch.cat([u, r, c], -1), rh, h
    outs = [torch.stack(v, 1) for v in (gates, resets, hiddens)]
    if squeeze:
        outs = [o[0] for o in outs]
    return _wrap(outs[0]), _wrap(outs[1]), _wrap(outs[2]), _wrap(outs[2].clone())


def lstm(input, h0=None, c0=None, weight=None, bias=None, use_peepholes=True, is_reverse=False, is_test=False,
         gate_activation="sigmoid", cell_activation="tanh", candidate_activation="tanh"):
    """The older LSTM operator: ``input`` holds x W_x already ([T, 4D] or [B, T, 4D]; columns candidate | input | forget |
    output), ``weight`` [D, 4D] in the same column order, ``bias`` [1, 4D], or [1, 7D] with the peephole vectors
    (W_ic, W_fc, W_oc) appended.  -> (hidden, cell, batch_gate, batch_cell_pre_act)."""
    xin, squeeze = _as_batch(_t(input))
    w = _t(weight)
    D = w.shape[0]
    peep = None
    if bias is not None:
        b = _t(bias).reshape(-1)
        xin = xin + b[:4 * D].reshape(1, 1, -1)
        if use_peepholes and b.numel() >= 7 * D:
            peep = b[4 * D:5 * D], b[5 * D:6 * D], b[6 * D:7 * D]
    B, T, _ = xin.shape
    h = _t(h0).reshape(B, D) if h0 is not None else xin.new_zeros(B, D)
    c = _t(c0).reshape(B, D) if c0 is not None else xin.new_zeros(B, D)
    ga, cella, canda = _ACT[gate_activation], _ACT[cell_activation], _ACT[candidate_activation]
    hs, cs, gs, pre = [None] * T, [None] * T, [None] * T, [None] * T
    for t in (range(T - 1, -1, -1) if is_reverse else range(T)):
        g = xin[:, t] + h @ w
        gc, gi, gf, go = g.chunk(4, -1)
        if peep is not None:
            gi, gf = gi + peep[0] * c, gf + peep[1] * c
        i, f, cand = ga(gi), ga(gf), canda(gc)
        c = f * c + i * cand
        if peep is not None:
            go = go + peep[2] * c
        o = ga(go)
        pre[t] = c
        h = o * cella(c)
        hs[t], cs[t], gs[t] = h, c, torch.cat([cand, i, f, o], -1)
    outs = [torch.stack(v, 1) for v in (hs, cs, gs, pre)]
    if squeeze:
        outs = [o[0] for o in outs]
    return tuple(_wrap(o) for o in outs)


# --------------------------------------------------------------------------------------------------------- detection
def _iou_one_to_many(box, boxes, normalized):
    off = 0.0 if normalized else 1.0
    x1, y1 = torch.maximum(box[0], boxes[:, 0]), torch.maximum(box[1], boxes[:, 1])
    x2, y2 = torch.minimum(box[2], boxes[:, 2]), torch.minimum(box[3], boxes[:, 3])
    inter = (x2 - x1 + off).clamp(min=0) * (y2 - y1 + off).clamp(min=0)
    area = lambda b: (b[..., 2] - b[..., 0] + off) * (b[..., 3] - b[..., 1] + off)
    return inter / (area(box) + area(boxes) - inter).clamp(min=1e-10)


def _nms_class(boxes, scores, score_threshold, nms_top_k, nms_threshold, nms_eta, normalized):
    """Indices kept for one class, best first; the overlap limit shrinks by ``nms_eta`` after each kept box while it
    stays above 0.5 (adaptive NMS)."""
    cand = torch.nonzero(scores > score_threshold).flatten()
    if cand.numel() == 0:
        return []
    order = cand[torch.argsort(scores[cand], descending=True, stable=True)]
    if nms_top_k > -1:
        order = order[:nms_top_k]
    keep, thr = [], float(nms_threshold)
    for idx in order.tolist():
        if keep and bool((_iou_one_to_many(boxes[idx], boxes[keep], normalized) > thr).any()):
            continue
        keep.append(idx)
        if nms_eta < 1.0 and thr > 0.5:
            thr *= nms_eta
    return keep


def multiclass_nms3(bboxes, scores, rois_num=None, score_threshold=0.05, nms_top_k=-1, keep_top_k=-1, nms_threshold=0.3,
                    normalized=True, nms_eta=1.0, background_label=0):
    """Per image and class: score filter, top ``nms_top_k``, NMS; then the best ``keep_top_k`` of the image.
    ``bboxes`` [N, M, 4] with ``scores`` [N, C, M]; or, with ``rois_num`` [N], ``bboxes`` [M, C, 4] and ``scores``
    [M, C] of all images concatenated.  -> (out [K, 6] rows (label, score, x1, y1, x2, y2), index [K, 1] into the
    flattened boxes, nms_rois_num [N] int32)."""
    bb, sc = _t(bboxes).float(), _t(scores).float()
    dev = bb.device
    bb_c, sc_c = bb.cpu(), sc.cpu()
    images = []
    if rois_num is not None:
        counts = _t(rois_num).cpu().tolist()
        start = 0
        for n in counts:
            images.append((bb_c[start:start + n], sc_c[start:start + n].t(), start, True))      # boxes [n, C, 4], scores [C, n]
            start += n
    else:
        M = bb_c.shape[1]
        for i in range(bb_c.shape[0]):
            images.append((bb_c[i], sc_c[i], i * M, False))
    rows, index, nums = [], [], []
    for boxes, s, base, per_class_boxes in images:
        found = []
        for cls in range(s.shape[0]):
            if cls == background_label:
                continue
            cb = boxes[:, cls] if per_class_boxes else boxes
            for k in _nms_class(cb, s[cls], score_threshold, nms_top_k, nms_threshold, nms_eta, normalized):
                found.append((float(s[cls, k]), cls, k, cb[k]))
        if keep_top_k > -1 and len(found) > keep_top_k:
            found = sorted(found, key=lambda f: -f[0])[:keep_top_k]
            found.sort(key=lambda f: f[1])                          # rows stay grouped by class, as produced
        for score, cls, k, box in found:
            rows.append(torch.cat([torch.tensor([float(cls), score]), box]))
            index.append(base + k)
        nums.append(len(found))
    out = torch.stack(rows) if rows else torch.zeros(0, 6)
    return (_wrap(out.to(dev)), _wrap(torch.tensor(index, dtype=torch.int32).reshape(-1, 1).to(dev)),
            _wrap(torch.tensor(nums, dtype=torch.int32).to(dev)))


def yolo_box_head(x, anchors, class_num):
    """Activation stage of a YOLO head on [N, A * (5 + C), H, W]: sigmoid on centre offsets, objectness and class
    scores, exp on width / height; the layout is unchanged."""
    t = _t(x)
    N, _, H, W = t.shape
    A = len(anchors) // 2
    v = t.reshape(N, A, 5 + class_num, H, W)
    out = torch.cat([torch.sigmoid(v[:, :, 0:2]), torch.exp(v[:, :, 2:4]), torch.sigmoid(v[:, :, 4:])], 2)
    return _wrap(out.reshape_as(t))


def yolo_box_post(boxes0, boxes1, boxes2, image_shape, image_scale, anchors0, anchors1, anchors2, class_num, conf_thresh,
                  downsample_ratio0, downsample_ratio1, downsample_ratio2, clip_bbox=True, scale_x_y=1.0, nms_threshold=0.45):
    """Decode three activated YOLO heads (outputs of ``yolo_box_head``) to image coordinates, drop boxes under
    ``conf_thresh`` and suppress overlaps among boxes of the same best class.  Rows: (class, objectness, x1, y1, x2,
    y2), ordered by class then class probability; a suppressed box stays in the list with objectness 0, as in the
    reference kernel.  -> (out [K, 6] - one zero row when nothing passes -, nms_rois_num [N] int32)."""
    heads = [(_t(b).float().cpu(), list(a), d) for b, a, d in ((boxes0, anchors0, downsample_ratio0),
                                                               (boxes1, anchors1, downsample_ratio1),
                                                               (boxes2, anchors2, downsample_ratio2))]
    shp, scl = _t(image_shape).float().cpu(), _t(image_scale).float().cpu()
    dev = _t(boxes0).device
    N = shp.shape[0]
    rows, nums = [], []
    for n in range(N):
        pic_h, pic_w = float(shp[n, 0] / scl[n, 0]), float(shp[n, 1] / scl[n, 1])
        dets = []
        for t, anchors, ratio in heads:
            A = len(anchors) // 2
            _, _, H, W = t.shape
            v = t[n].reshape(A, 5 + class_num, H, W)
            obj = v[:, 4]
            sel = torch.nonzero(obj >= conf_thresh)
            if sel.numel() == 0:
                continue
            a, gy, gx = sel[:, 0], sel[:, 1], sel[:, 2]
            aw = torch.tensor(anchors[0::2], dtype=torch.float32)[a]
            ah = torch.tensor(anchors[1::2], dtype=torch.float32)[a]
            cx = (v[a, 0, gy, gx] + gx) * pic_w / W
            cy = (v[a, 1, gy, gx] + gy) * pic_h / H
            bw = v[a, 2, gy, gx] * aw * pic_w / (ratio * W)
            bh = v[a, 3, gy, gx] * ah * pic_h / (ratio * H)
            x1, y1 = (cx - bw / 2).clamp(min=0), (cy - bh / 2).clamp(min=0)
            x2, y2 = (cx + bw / 2).clamp(max=pic_w - 1), (cy + bh / 2).clamp(max=pic_h - 1)
            o = obj[a, gy, gx]
            probs = v[a, 5:, gy, gx] * o.unsqueeze(-1)
            best_p, best_c = torch.max(probs, -1)
            best_c = torch.where(best_p > 0, best_c, torch.full_like(best_c, -1))
            dets.append(torch.stack([best_c.float(), o, x1, y1, x2, y2, best_p], 1))
        if not dets:
            nums.append(0)
            continue
        d = torch.cat(dets)
        order = sorted(range(d.shape[0]), key=lambda i: (float(d[i, 0]), -float(d[i, 6])))
        d = d[order]
        for i in range(d.shape[0]):
            if d[i, 1] == 0:
                continue
            for j in range(i + 1, d.shape[0]):
                if d[j, 0] != d[i, 0]:
                    break
                if d[j, 1] != 0 and float(_iou_one_to_many(d[i, 2:6], d[j:j + 1, 2:6], True)) > nms_threshold:
                    d[j, 1] = 0
        rows.append(d[:, :6])
        nums.append(d.shape[0])
    out = torch.cat(rows) if rows else torch.zeros(1, 6)
    return _wrap(out.to(dev)), _wrap(torch.tensor(nums, dtype=torch.int32).to(dev))


def collect_fpn_proposals(multi_level_rois, multi_level_scores, multi_level_rois_num=None, post_nms_topn=-1):
    """Merge the proposals of all pyramid levels, keep the ``post_nms_topn`` best by score and return them grouped by
    image.  Without per-level counts everything belongs to one image.  -> (fpn_rois [K, 4], rois_num [N] int32)."""
    rois = torch.cat([_t(r) for r in multi_level_rois])
    scores = torch.cat([_t(s).reshape(-1) for s in multi_level_scores])
    if multi_level_rois_num:
        batch = torch.cat([torch.repeat_interleave(torch.arange(_t(c).numel(), device=rois.device), _t(c).to(rois.device).long())
                           for c in multi_level_rois_num])
        n_img = _t(multi_level_rois_num[0]).numel()
    else:
        batch = torch.zeros(rois.shape[0], dtype=torch.long, device=rois.device)
        n_img = 1
    k = rois.shape[0] if post_nms_topn < 0 else min(post_nms_topn, rois.shape[0])
    top = torch.argsort(scores, descending=True, stable=True)[:k]
    top = top[torch.argsort(batch[top], stable=True)]                  # by image, score order kept inside an image
    nums = torch.bincount(batch[top], minlength=n_img).to(torch.int32)
    return _wrap(rois[top]), _wrap(nums)


def correlation(input1, input2, pad_size, kernel_size, max_displacement, stride1, stride2, corr_type_multiply=1):
    """Cost volume of optical-flow networks: for each displacement (dy, dx) on a grid of step ``stride2`` within
    ``max_displacement``, the mean over channels and a ``kernel_size`` window of input1 * shifted input2.
    NCHW -> [N, (2 * (max_displacement // stride2) + 1)^2, H', W']."""
    a, b = _t(input1), _t(input2)
    N, C, H, W = a.shape
    kr = (kernel_size - 1) // 2
    dr = max_displacement // stride2
    border = max_displacement + kr
    ph, pw = H + 2 * pad_size, W + 2 * pad_size
    oh, ow = math.ceil((ph - 2 * border) / stride1), math.ceil((pw - 2 * border) / stride1)
    if oh <= 0 or ow <= 0:
        raise ValueError("correlation: the padded input is smaller than the displacement border")
    # extra margin so that shifted windows never leave the buffer; the margin reads as zero like the padding
    m = max_displacement + kr
    ap, bp = TF.pad(a, [pad_size + m] * 4), TF.pad(b, [pad_size + m] * 4)
    ys = torch.arange(oh, device=a.device) * stride1 + max_displacement + m
    xs = torch.arange(ow, device=a.device) * stride1 + max_displacement + m
    outs = []
    for tj in range(-dr, dr + 1):
        for ti in range(-dr, dr + 1):
            acc = a.new_zeros(N, oh, ow)
            for j in range(-kr, kr + 1):
                for i in range(-kr, kr + 1):
                    p1 = ap[:, :, (ys + j)[:, None], (xs + i)[None, :]]
                    p2 = bp[:, :, (ys + j + tj * stride2)[:, None], (xs + i + ti * stride2)[None, :]]
                    acc = acc + (p1 * p2).sum(1)
            outs.append(acc / (kernel_size * kernel_size * C))
    return _wrap(torch.stack(outs, 1))
