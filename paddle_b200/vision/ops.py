"""``paddle.vision.ops`` (python/paddle/vision/ops.py; kernels paddle/phi/kernels/gpu/{nms,roi_align,roi_pool,
deformable_conv,yolo_box,prior_box,box_coder}_kernel.cu): detection operators written as tensor arithmetic
(they run on any device; no graphics stack is involved)."""
from __future__ import annotations

import math

import torch

from .._core.tensor import as_tensor
from ..nn.layer.layers import Layer

__all__ = ["nms", "roi_align", "roi_pool", "psroi_pool", "deform_conv2d", "DeformConv2D", "RoIAlign", "RoIPool",
           "PSRoIPool", "box_coder", "prior_box", "yolo_box", "yolo_loss", "generate_proposals", "distribute_fpn_proposals",
           "matrix_nms", "read_file", "decode_jpeg"]


def _p(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def _iou(a, b):
    area = lambda t: (t[:, 2] - t[:, 0]).clamp(min=0) * (t[:, 3] - t[:, 1]).clamp(min=0)   # noqa: E731
    lt = torch.max(a[:, None, :2], b[None, :, :2])
    rb = torch.min(a[:, None, 2:], b[None, :, 2:])
    inter = (rb - lt).clamp(min=0).prod(-1)
    return inter / (area(a)[:, None] + area(b)[None] - inter + 1e-10)


def nms(boxes, iou_threshold=0.3, scores=None, category_idxs=None, categories=None, top_k=None):
    boxes = _p(boxes).float()
    n = boxes.shape[0]
    order = torch.argsort(_p(scores).float(), descending=True) if scores is not None else torch.arange(n)
    if category_idxs is not None:
        # boxes of different categories never suppress each other: shift them apart
        off = _p(category_idxs).float() * (boxes.max() + 1)
        work = boxes + off[:, None]
    else:
        work = boxes
    iou = _iou(work[order], work[order])
    keep = []
    alive = torch.ones(n, dtype=torch.bool)
    for i in range(n):
        if not alive[i]:
            continue
        keep.append(int(order[i]))
        alive &= ~(iou[i] > iou_threshold)
        alive[i] = False
    keep = torch.tensor(keep, dtype=torch.int64)
    return as_tensor(keep[:top_k] if top_k else keep)


def _bilinear(feat, y, x):
    """feat [C, H, W]; y, x arbitrary-shaped float coordinates -> [C, *shape] (zero outside)."""
    C, H, W = feat.shape
    valid = (y > -1) & (y < H) & (x > -1) & (x < W)
    y, x = y.clamp(0, H - 1), x.clamp(0, W - 1)
    y0, x0 = y.floor().long(), x.floor().long()
    y1, x1 = (y0 + 1).clamp(max=H - 1), (x0 + 1).clamp(max=W - 1)
    ly, lx = y - y0, x - x0
    v = (feat[:, y0, x0] * (1 - ly) * (1 - lx) + feat[:, y0, x1] * (1 - ly) * lx +
         feat[:, y1, x0] * ly * (1 - lx) + feat[:, y1, x1] * ly * lx)
    return v * valid


def _bilinear_zero(feat, y, x):
    """Bilinear sample with zero padding: corners outside the image contribute nothing (deformable convolution)."""
    C, H, W = feat.shape
    y0, x0 = y.floor(), x.floor()
    ly, lx = y - y0, x - x0
    out = 0
    for dy, wy in ((0, 1 - ly), (1, ly)):
        for dx, wx in ((0, 1 - lx), (1, lx)):
            yi, xi = (y0 + dy).long(), (x0 + dx).long()
            ok = (yi >= 0) & (yi < H) & (xi >= 0) & (xi < W)
            out = out + feat[:, yi.clamp(0, H - 1), xi.clamp(0, W - 1)] * (wy * wx * ok)
    return out


def roi_align(x, boxes, boxes_num, output_size, spatial_scale=1.0, sampling_ratio=-1, aligned=True, name=None):
    x, boxes = _p(x), _p(boxes).float()
    oh, ow = (output_size, output_size) if isinstance(output_size, int) else output_size
    img = torch.repeat_interleave(torch.arange(len(boxes_num)), _p(boxes_num).long())
    off = 0.5 if aligned else 0.0
    outs = []
    for b, box in zip(img.tolist(), boxes):
        x1, y1, x2, y2 = (box * spatial_scale - off).tolist()
        rw, rh = x2 - x1, y2 - y1
        if not aligned:
            rw, rh = max(rw, 1.0), max(rh, 1.0)
        bw, bh = rw / ow, rh / oh
        sy = sampling_ratio if sampling_ratio > 0 else max(int(math.ceil(rh / oh)), 1)
        sx = sampling_ratio if sampling_ratio > 0 else max(int(math.ceil(rw / ow)), 1)
        iy = (torch.arange(oh)[:, None] * bh + y1 + (torch.arange(sy)[None] + 0.5) * bh / sy).reshape(-1)
        ix = (torch.arange(ow)[:, None] * bw + x1 + (torch.arange(sx)[None] + 0.5) * bw / sx).reshape(-1)
        yy, xx = torch.meshgrid(iy, ix, indexing="ij")
        v = _bilinear(x[b].float(), yy.to(x.device), xx.to(x.device))
        outs.append(v.reshape(-1, oh, sy, ow, sx).mean((2, 4)))
    return as_tensor(torch.stack(outs).to(x.dtype) if outs else x.new_zeros((0, x.shape[1], oh, ow)))


def roi_pool(x, boxes, boxes_num, output_size, spatial_scale=1.0, name=None):
    x, boxes = _p(x), _p(boxes).float()
    oh, ow = (output_size, output_size) if isinstance(output_size, int) else output_size
    img = torch.repeat_interleave(torch.arange(len(boxes_num)), _p(boxes_num).long())
    H, W = x.shape[-2:]
    outs = []
    for b, box in zip(img.tolist(), boxes):
        x1, y1, x2, y2 = [int(round(v * spatial_scale)) for v in box.tolist()]
        rh, rw = max(y2 - y1 + 1, 1), max(x2 - x1 + 1, 1)
        o = x.new_zeros((x.shape[1], oh, ow))
        for i in range(oh):
            for j in range(ow):
                hs, he = min(max(y1 + int(math.floor(i * rh / oh)), 0), H), min(max(y1 + int(math.ceil((i + 1) * rh / oh)), 0), H)
                ws, we = min(max(x1 + int(math.floor(j * rw / ow)), 0), W), min(max(x1 + int(math.ceil((j + 1) * rw / ow)), 0), W)
                if he > hs and we > ws:
                    o[:, i, j] = x[b, :, hs:he, ws:we].amax((-2, -1))
        outs.append(o)
    return as_tensor(torch.stack(outs) if outs else x.new_zeros((0, x.shape[1], oh, ow)))


def psroi_pool(x, boxes, boxes_num, output_size, spatial_scale=1.0, name=None):
    x, boxes = _p(x), _p(boxes).float()
    oh, ow = (output_size, output_size) if isinstance(output_size, int) else output_size
    C = x.shape[1] // (oh * ow)
    img = torch.repeat_interleave(torch.arange(len(boxes_num)), _p(boxes_num).long())
    H, W = x.shape[-2:]
    outs = []
    for b, box in zip(img.tolist(), boxes):
        x1, y1, x2, y2 = (box * spatial_scale).tolist()
        rh, rw = max(y2 - y1, 0.1), max(x2 - x1, 0.1)
        o = x.new_zeros((C, oh, ow))
        for i in range(oh):
            for j in range(ow):
                hs, he = int(math.floor(y1 + i * rh / oh)), int(math.ceil(y1 + (i + 1) * rh / oh))
                ws, we = int(math.floor(x1 + j * rw / ow)), int(math.ceil(x1 + (j + 1) * rw / ow))
                hs, he, ws, we = max(hs, 0), min(he, H), max(ws, 0), min(we, W)
                if he > hs and we > ws:
                    ch = torch.arange(C) * oh * ow + i * ow + j
                    o[:, i, j] = x[b, ch, hs:he, ws:we].mean((-2, -1))
        outs.append(o)
    return as_tensor(torch.stack(outs) if outs else x.new_zeros((0, C, oh, ow)))


def deform_conv2d(x, offset, weight, bias=None, stride=1, padding=0, dilation=1, deformable_groups=1, groups=1,
                  mask=None, name=None):
    """Deformable convolution v1 (mask None) / v2: bilinear sampling at offset kernel taps, then a dense contraction."""
    x, offset, weight = _p(x), _p(offset), _p(weight)
    pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)   # noqa: E731
    (sh, sw), (ph, pw), (dh, dw) = pair(stride), pair(padding), pair(dilation)
    N, C, H, W = x.shape
    Co, Cg, kh, kw = weight.shape
    Ho = (H + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    Wo = (W + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    base_y = (torch.arange(Ho, device=x.device) * sh - ph)[:, None].float()
    base_x = (torch.arange(Wo, device=x.device) * sw - pw)[None, :].float()
    cols = x.new_zeros((N, C, kh * kw, Ho, Wo))
    cpg = C // deformable_groups
    off = offset.reshape(N, deformable_groups, kh * kw, 2, Ho, Wo).float()
    msk = _p(mask).reshape(N, deformable_groups, kh * kw, Ho, Wo).float() if mask is not None else None
    for n in range(N):
        for g in range(deformable_groups):
            feat = x[n, g * cpg:(g + 1) * cpg].float()
            for k in range(kh * kw):
                yy = base_y + (k // kw) * dh + off[n, g, k, 0]
                xx = base_x + (k % kw) * dw + off[n, g, k, 1]
                v = _bilinear_zero(feat, yy, xx)
                if msk is not None:
                    v = v * msk[n, g, k]
                cols[n, g * cpg:(g + 1) * cpg, k] = v.to(x.dtype)
    cols = cols.reshape(N, groups, (C // groups) * kh * kw, Ho * Wo)
    w = weight.reshape(groups, Co // groups, Cg * kh * kw)
    out = torch.einsum("gok,ngkl->ngol", w.float(), cols.float()).reshape(N, Co, Ho, Wo).to(x.dtype)
    if bias is not None:
        out = out + _p(bias).reshape(1, -1, 1, 1)
    return as_tensor(out)


class DeformConv2D(Layer):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, deformable_groups=1,
                 groups=1, weight_attr=None, bias_attr=None):
        super().__init__()
        ks = (kernel_size, kernel_size) if isinstance(kernel_size, int) else tuple(kernel_size)
        self.weight = self.create_parameter([out_channels, in_channels // groups, *ks], attr=weight_attr)
        self.bias = None if bias_attr is False else self.create_parameter([out_channels], attr=bias_attr, is_bias=True)
        self._cfg = (stride, padding, dilation, deformable_groups, groups)

    def forward(self, x, offset, mask=None):
        s, p, d, dg, g = self._cfg
        return deform_conv2d(x, offset, self.weight, self.bias, s, p, d, dg, g, mask)


class RoIAlign(Layer):
    def __init__(self, output_size, spatial_scale=1.0):
        super().__init__()
        self.output_size, self.spatial_scale = output_size, spatial_scale

    def forward(self, x, boxes, boxes_num, aligned=True):
        return roi_align(x, boxes, boxes_num, self.output_size, self.spatial_scale, aligned=aligned)


class RoIPool(Layer):
    def __init__(self, output_size, spatial_scale=1.0):
        super().__init__()
        self.output_size, self.spatial_scale = output_size, spatial_scale

    def forward(self, x, boxes, boxes_num):
        return roi_pool(x, boxes, boxes_num, self.output_size, self.spatial_scale)


class PSRoIPool(Layer):
    def __init__(self, output_size, spatial_scale=1.0):
        super().__init__()
        self.output_size, self.spatial_scale = output_size, spatial_scale

    def forward(self, x, boxes, boxes_num):
        return psroi_pool(x, boxes, boxes_num, self.output_size, self.spatial_scale)


def box_coder(prior_box, prior_box_var, target_box, code_type="encode_center_size", box_normalized=True, axis=0, name=None):
    pb, tb = _p(prior_box).float(), _p(target_box).float()
    var = _p(prior_box_var).float() if isinstance(prior_box_var, torch.Tensor) else \
        torch.tensor(prior_box_var if prior_box_var is not None else [1.0] * 4).float()
    norm = 0.0 if box_normalized else 1.0
    pw, ph = pb[:, 2] - pb[:, 0] + norm, pb[:, 3] - pb[:, 1] + norm
    px, py = pb[:, 0] + pw / 2, pb[:, 1] + ph / 2
    if code_type == "encode_center_size":
        tw, th = tb[:, 2] - tb[:, 0] + norm, tb[:, 3] - tb[:, 1] + norm
        tx, ty = tb[:, 0] + tw / 2, tb[:, 1] + th / 2
        out = torch.stack([(tx[:, None] - px[None]) / pw[None], (ty[:, None] - py[None]) / ph[None],
                           torch.log(tw[:, None] / pw[None]), torch.log(th[:, None] / ph[None])], -1)
        return as_tensor(out / (var if var.dim() == 1 else var[None]))
    v = var if var.dim() == 1 else (var[None] if axis == 0 else var[:, None])
    shp = (1, -1) if axis == 0 else (-1, 1)
    pw, ph, px, py = (t.reshape(shp) for t in (pw, ph, px, py))
    d = tb * v
    cx, cy = d[..., 0] * pw + px, d[..., 1] * ph + py
    w, h = torch.exp(d[..., 2]) * pw, torch.exp(d[..., 3]) * ph
    return as_tensor(torch.stack([cx - w / 2, cy - h / 2, cx + w / 2 - norm, cy + h / 2 - norm], -1))


def prior_box(input, image, min_sizes, max_sizes=None, aspect_ratios=(1.0,), variance=(0.1, 0.1, 0.2, 0.2), flip=False,
              clip=False, steps=(0.0, 0.0), offset=0.5, min_max_aspect_ratios_order=False, name=None):
    H, W = input.shape[-2:]
    IH, IW = image.shape[-2:]
    sw = steps[0] or IW / W
    sh = steps[1] or IH / H
    ars = [1.0]
    for a in aspect_ratios:
        if all(abs(a - b) > 1e-6 for b in ars):
            ars.append(a)
            if flip:
                ars.append(1.0 / a)
    boxes = []
    for i in range(H):
        for j in range(W):
            cx, cy = (j + offset) * sw, (i + offset) * sh
            for k, ms in enumerate(min_sizes):
                cell = [(ms, ms)]
                if max_sizes:
                    s = math.sqrt(ms * max_sizes[k])
                    cell.append((s, s))
                cell += [(ms * math.sqrt(a), ms / math.sqrt(a)) for a in ars if abs(a - 1.0) > 1e-6]
                for bw, bh in cell:
                    boxes.append([(cx - bw / 2) / IW, (cy - bh / 2) / IH, (cx + bw / 2) / IW, (cy + bh / 2) / IH])
    b = torch.tensor(boxes).reshape(H, W, -1, 4)
    if clip:
        b = b.clamp(0, 1)
    return as_tensor(b), as_tensor(torch.tensor(variance).expand_as(b).clone())


def yolo_box(x, img_size, anchors, class_num, conf_thresh, downsample_ratio, clip_bbox=True, name=None, scale_x_y=1.0,
             iou_aware=False, iou_aware_factor=0.5):
    x, img_size = _p(x).float(), _p(img_size).float()
    N, _, H, W = x.shape
    A = len(anchors) // 2
    x = x.reshape(N, A, 5 + class_num, H, W)
    gy, gx = torch.meshgrid(torch.arange(H), torch.arange(W), indexing="ij")
    bias = -0.5 * (scale_x_y - 1.0)
    cx = (torch.sigmoid(x[:, :, 0]) * scale_x_y + bias + gx) / W
    cy = (torch.sigmoid(x[:, :, 1]) * scale_x_y + bias + gy) / H
    aw = torch.tensor(anchors[0::2]).reshape(1, A, 1, 1).float()
    ah = torch.tensor(anchors[1::2]).reshape(1, A, 1, 1).float()
    bw = torch.exp(x[:, :, 2]) * aw / (W * downsample_ratio)
    bh = torch.exp(x[:, :, 3]) * ah / (H * downsample_ratio)
    conf = torch.sigmoid(x[:, :, 4])
    ih, iw = img_size[:, 0].reshape(N, 1, 1, 1), img_size[:, 1].reshape(N, 1, 1, 1)
    boxes = torch.stack([(cx - bw / 2) * iw, (cy - bh / 2) * ih, (cx + bw / 2) * iw, (cy + bh / 2) * ih], -1)
    if clip_bbox:
        boxes = torch.stack([boxes[..., 0].clamp(min=0), boxes[..., 1].clamp(min=0),
                             torch.minimum(boxes[..., 2], iw - 1), torch.minimum(boxes[..., 3], ih - 1)], -1)
    keep = (conf >= conf_thresh).float()
    scores = (torch.sigmoid(x[:, :, 5:]) * (conf * keep).unsqueeze(2)).permute(0, 1, 3, 4, 2)
    boxes = boxes * keep.unsqueeze(-1)
    return as_tensor(boxes.reshape(N, -1, 4)), as_tensor(scores.reshape(N, -1, class_num))


def _sce(x, label):
    """Sigmoid cross entropy on a logit, log(1 + e^x) - x * label (softplus keeps it stable and smooth at 0)."""
    return torch.nn.functional.softplus(x) - x * label


def yolo_loss(x, gt_box, gt_label, anchors, anchor_mask, class_num, ignore_thresh, downsample_ratio, gt_score=None,
              use_label_smooth=True, name=None, scale_x_y=1.0):
    """YOLOv3 training loss of one detection head (python/paddle/vision/ops.py ``yolo_loss``; kernel
    paddle/phi/kernels/cpu/yolo_loss_kernel.cc).  ``x`` [N, len(anchor_mask) * (5 + class_num), H, W] raw head output;
    ``gt_box`` [N, B, 4] normalised (cx, cy, w, h), rows with w or h <= 0 are padding; ``gt_label`` [N, B].  Per image:

    * every prediction whose decoded box overlaps some ground truth by more than ``ignore_thresh`` is left out of the
      objectness loss unless it is a positive;
    * every ground truth picks, among ALL anchors, the one whose shape fits best; when that anchor belongs to this head
      (``anchor_mask``) the cell holding the box centre becomes a positive: sigmoid cross entropy on the centre offsets,
      L1 on the log sizes, both weighted by ``(2 - w * h) * score``; class sigmoid cross entropy (smoothed targets
      ``1 - 1 / class_num`` / ``1 / class_num`` with ``use_label_smooth``) weighted by ``score``; objectness target
      ``score`` (``gt_score``, 1 by default);
    * all other kept predictions have objectness target 0.
    -> loss [N]."""
    xt = _p(x)
    xt = xt if xt.dtype == torch.float64 else xt.float()
    gb, gl = _p(gt_box).to(xt.dtype), _p(gt_label).long()
    N, _, H, W = xt.shape
    an_num, mask_num = len(anchors) // 2, len(anchor_mask)
    B = gb.shape[1]
    gs = _p(gt_score).to(xt.dtype) if gt_score is not None else torch.ones(N, B, dtype=xt.dtype)
    input_size = downsample_ratio * H
    v = xt.reshape(N, mask_num, 5 + class_num, H, W)
    bias = -0.5 * (scale_x_y - 1.0)
    pos, neg = (1.0 - 1.0 / class_num, 1.0 / class_num) if use_label_smooth else (1.0, 0.0)
    aw_all = torch.tensor(anchors[0::2], dtype=xt.dtype)
    ah_all = torch.tensor(anchors[1::2], dtype=xt.dtype)
    # decoded prediction boxes (no gradient: they only decide which predictions are ignored)
    with torch.no_grad():
        gx = torch.arange(W, dtype=xt.dtype).reshape(1, 1, 1, W)
        gy = torch.arange(H, dtype=xt.dtype).reshape(1, 1, H, 1)
        maw = aw_all[list(anchor_mask)].reshape(1, mask_num, 1, 1)
        mah = ah_all[list(anchor_mask)].reshape(1, mask_num, 1, 1)
        px = (gx + torch.sigmoid(v[:, :, 0]) * scale_x_y + bias) / W
        py = (gy + torch.sigmoid(v[:, :, 1]) * scale_x_y + bias) / H
        pw = torch.exp(v[:, :, 2]) * maw / input_size
        ph = torch.exp(v[:, :, 3]) * mah / input_size
        valid = (gb[..., 2] > 0) & (gb[..., 3] > 0)                                   # [N, B]

        def iou_cxcywh(ax, ay, aw_, ah_, bx, by, bw, bh):
            l = torch.maximum(ax - aw_ / 2, bx - bw / 2)
            r = torch.minimum(ax + aw_ / 2, bx + bw / 2)
            t = torch.maximum(ay - ah_ / 2, by - bh / 2)
            b = torch.minimum(ay + ah_ / 2, by + bh / 2)
            inter = (r - l).clamp(min=0) * (b - t).clamp(min=0)
            return inter / (aw_ * ah_ + bw * bh - inter).clamp(min=1e-10)
        e = lambda t: t.unsqueeze(-1)                                                  # noqa: E731
        g = lambda t: t.reshape(N, 1, 1, 1, B)                                         # noqa: E731
        ious = iou_cxcywh(e(px), e(py), e(pw), e(ph), g(gb[..., 0]), g(gb[..., 1]), g(gb[..., 2]), g(gb[..., 3]))
        ious = torch.where(valid.reshape(N, 1, 1, 1, B), ious, torch.zeros_like(ious))
        obj_mask = torch.where(ious.max(-1).values > ignore_thresh, -torch.ones_like(px), torch.zeros_like(px))   # [N, A, H, W]
    loss = xt.new_zeros(N)
    for i in range(N):
        for t in range(B):
            if not bool(valid[i, t]):
                continue
            bx, by, bw, bh = (float(c) for c in gb[i, t])
            gi, gj = int(bx * W), int(by * H)
            # best anchor by shape overlap (both boxes centred at the origin)
            iw = torch.minimum(aw_all / input_size, torch.tensor(bw, dtype=xt.dtype))
            ih = torch.minimum(ah_all / input_size, torch.tensor(bh, dtype=xt.dtype))
            inter = iw * ih
            shape_iou = inter / (aw_all * ah_all / input_size ** 2 + bw * bh - inter)
            best_n = int(torch.argmax(shape_iou))
            if best_n not in list(anchor_mask):
                continue
            a = list(anchor_mask).index(best_n)
            score = gs[i, t]
            tx, ty = bx * W - gi, by * H - gj
            tw = math.log(bw * input_size / anchors[2 * best_n])
            th = math.log(bh * input_size / anchors[2 * best_n + 1])
            scale = (2.0 - bw * bh) * score
            cell = v[i, a, :, gj, gi]
            loss[i] = loss[i] + (_sce(cell[0], tx) + _sce(cell[1], ty) + (cell[2] - tw).abs() + (cell[3] - th).abs()) * scale
            obj_mask[i, a, gj, gi] = score
            target = torch.full((class_num,), neg, dtype=xt.dtype)
            target[int(gl[i, t])] = pos
            loss[i] = loss[i] + (_sce(cell[5:], target) * score).sum()
    obj_logit = v[:, :, 4]
    pos_part = torch.where(obj_mask > 1e-6, _sce(obj_logit, torch.ones_like(obj_logit)) * obj_mask, torch.zeros_like(obj_logit))
    neg_part = torch.where((obj_mask <= 1e-6) & (obj_mask > -0.5), _sce(obj_logit, torch.zeros_like(obj_logit)), torch.zeros_like(obj_logit))
    loss = loss + (pos_part + neg_part).sum((1, 2, 3))
    return as_tensor(loss.to(_p(x).dtype))


def matrix_nms(bboxes, scores, score_threshold, post_threshold, nms_top_k, keep_top_k, use_gaussian=False,
               gaussian_sigma=2.0, background_label=0, normalized=True, return_index=False, return_rois_num=True, name=None):
    bboxes, scores = _p(bboxes).float(), _p(scores).float()
    outs, idxs, nums = [], [], []
    for n in range(bboxes.shape[0]):
        res = []
        for c in range(scores.shape[1]):
            if c == background_label:
                continue
            sc = scores[n, c]
            sel = torch.nonzero(sc > score_threshold).reshape(-1)
            if sel.numel() == 0:
                continue
            order = sel[torch.argsort(sc[sel], descending=True)][:nms_top_k if nms_top_k > 0 else None]
            b, s = bboxes[n, order], sc[order]
            iou = _iou(b, b).triu(1)
            cmax = iou.max(0).values
            decay = (torch.exp(-(iou ** 2 - cmax[:, None] ** 2) / gaussian_sigma) if use_gaussian
                     else (1 - iou) / (1 - cmax[:, None])).min(0).values
            s2 = s * decay
            ok = s2 > post_threshold
            for i in torch.nonzero(ok).reshape(-1).tolist():
                res.append((float(s2[i]), c, b[i], int(order[i]) + n * bboxes.shape[1]))
        res.sort(key=lambda t: -t[0])
        res = res[:keep_top_k if keep_top_k > 0 else None]
        nums.append(len(res))
        for s, c, b, i in res:
            outs.append(torch.cat([torch.tensor([float(c), s]), b]))
            idxs.append(i)
    out = torch.stack(outs) if outs else torch.zeros((0, 6))
    ret = [as_tensor(out)]
    if return_index:
        ret.append(as_tensor(torch.tensor(idxs, dtype=torch.int64).reshape(-1, 1)))
    if return_rois_num:
        ret.append(as_tensor(torch.tensor(nums, dtype=torch.int32)))
    return tuple(ret) if len(ret) > 1 else ret[0]


def generate_proposals(scores, bbox_deltas, img_size, anchors, variances, pre_nms_top_n=6000, post_nms_top_n=1000,
                       nms_thresh=0.5, min_size=0.1, eta=1.0, pixel_offset=False, return_rois_num=False, name=None):
    scores, deltas = _p(scores).float(), _p(bbox_deltas).float()
    anchors, variances = _p(anchors).float().reshape(-1, 4), _p(variances).float().reshape(-1, 4)
    N = scores.shape[0]
    rois, probs, nums = [], [], []
    off = 1.0 if pixel_offset else 0.0
    for n in range(N):
        s = scores[n].permute(1, 2, 0).reshape(-1)
        d = deltas[n].permute(1, 2, 0).reshape(-1, 4)
        order = torch.argsort(s, descending=True)[:pre_nms_top_n]
        s, d, a, v = s[order], d[order], anchors[order], variances[order]
        aw, ah = a[:, 2] - a[:, 0] + off, a[:, 3] - a[:, 1] + off
        ax, ay = a[:, 0] + aw / 2, a[:, 1] + ah / 2
        cx, cy = v[:, 0] * d[:, 0] * aw + ax, v[:, 1] * d[:, 1] * ah + ay
        w = torch.exp((v[:, 2] * d[:, 2]).clamp(max=math.log(1000 / 16))) * aw
        h = torch.exp((v[:, 3] * d[:, 3]).clamp(max=math.log(1000 / 16))) * ah
        box = torch.stack([cx - w / 2, cy - h / 2, cx + w / 2 - off, cy + h / 2 - off], -1)
        ih, iw = float(img_size[n][0]), float(img_size[n][1])
        box = torch.stack([box[:, 0].clamp(0, iw - off), box[:, 1].clamp(0, ih - off), box[:, 2].clamp(0, iw - off),
                           box[:, 3].clamp(0, ih - off)], -1)
        keep = ((box[:, 2] - box[:, 0] + off) >= min_size) & ((box[:, 3] - box[:, 1] + off) >= min_size)
        box, s = box[keep], s[keep]
        k = _p(nms(box, nms_thresh, s))[:post_nms_top_n]
        rois.append(box[k]), probs.append(s[k]), nums.append(k.numel())
    out = (as_tensor(torch.cat(rois)), as_tensor(torch.cat(probs).reshape(-1, 1)))
    return out + (as_tensor(torch.tensor(nums, dtype=torch.int32)),) if return_rois_num else out


def distribute_fpn_proposals(fpn_rois, min_level, max_level, refer_level, refer_scale, pixel_offset=False,
                             rois_num=None, name=None):
    rois = _p(fpn_rois).float()
    off = 1.0 if pixel_offset else 0.0
    scale = torch.sqrt(((rois[:, 2] - rois[:, 0] + off) * (rois[:, 3] - rois[:, 1] + off)).clamp(min=0))
    lvl = torch.floor(torch.log2(scale / refer_scale + 1e-8) + refer_level).clamp(min_level, max_level).long()
    multi, order = [], []
    for l in range(min_level, max_level + 1):
        idx = torch.nonzero(lvl == l).reshape(-1)
        multi.append(as_tensor(rois[idx]))
        order.append(idx)
    restore = torch.empty(rois.shape[0], dtype=torch.int64)
    restore[torch.cat(order)] = torch.arange(rois.shape[0])
    nums = [as_tensor(torch.tensor([o.numel()], dtype=torch.int32)) for o in order] if rois_num is not None else None
    return multi, as_tensor(restore.reshape(-1, 1)), nums


def read_file(filename, name=None):
    with open(filename, "rb") as f:
        return as_tensor(torch.frombuffer(bytearray(f.read()), dtype=torch.uint8))


def decode_jpeg(x, mode="unchanged", name=None):
    import io

    import numpy as np
    from PIL import Image
    img = Image.open(io.BytesIO(bytes(_p(x).tolist())))
    if mode == "gray":
        img = img.convert("L")
    elif mode == "rgb":
        img = img.convert("RGB")
    a = np.asarray(img)
    a = a[None] if a.ndim == 2 else a.transpose(2, 0, 1)
    return as_tensor(torch.from_numpy(a.copy()))
