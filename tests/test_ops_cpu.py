"""Table-driven operator tests: forward against NumPy, gradient against central differences (the reference's
per-op files such as test/legacy_test/test_elementwise_add_op.py, test_softmax_op.py, test_conv2d_op.py, ...)."""
import numpy as np
import pytest

import paddle_b200 as paddle
import paddle_b200.nn.functional as F
from op_test import check_grad, check_output

R = np.random.RandomState(0)


def f32(*shape, lo=-1.0, hi=1.0):
    return R.uniform(lo, hi, size=shape).astype(np.float32)


def _softmax(x, axis):
    e = np.exp(x - x.max(axis, keepdims=True))
    return e / e.sum(axis, keepdims=True)


def _conv2d_ref(x, w, b, stride, pad):
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    oh, ow = (h + 2 * pad - kh) // stride + 1, (wd + 2 * pad - kw) // stride + 1
    out = np.zeros((n, o, oh, ow))
    for i in range(oh):
        for j in range(ow):
            patch = xp[:, :, i * stride:i * stride + kh, j * stride:j * stride + kw]
            out[:, :, i, j] = np.einsum("nchw,ochw->no", patch, w)
    return out + b.reshape(1, -1, 1, 1)


def _layer_norm_ref(x, w, b, eps):
    m, v = x.mean(-1, keepdims=True), x.var(-1, keepdims=True)
    return (x - m) / np.sqrt(v + eps) * w + b


def _pool_ref(x, k, s, fn):
    n, c, h, w = x.shape
    oh, ow = (h - k) // s + 1, (w - k) // s + 1
    out = np.zeros((n, c, oh, ow))
    for i in range(oh):
        for j in range(ow):
            out[:, :, i, j] = fn(x[:, :, i * s:i * s + k, j * s:j * s + k], axis=(2, 3))
    return out


def _ce_ref(logits, label):
    p = _softmax(logits, -1)
    return -np.log(p[np.arange(len(label)), label]).mean()


def _gelu(x):
    from math import erf
    return 0.5 * x * (1 + np.vectorize(erf)(x / np.sqrt(2)))


A, B = f32(3, 4), f32(3, 4)
POS = f32(3, 4, lo=0.5, hi=2.0)
IDX = np.array([2, 0, 1], dtype=np.int64)

CASES = [
    # name, fn(**inputs), inputs, numpy reference, inputs to differentiate
    ("add_broadcast", lambda x, y: paddle.add(x, y), dict(x=A, y=f32(4)), lambda x, y: x + y, ["x", "y"]),
    ("subtract", lambda x, y: paddle.subtract(x, y), dict(x=A, y=B), lambda x, y: x - y, ["x", "y"]),
    ("multiply", lambda x, y: paddle.multiply(x, y), dict(x=A, y=B), lambda x, y: x * y, ["x", "y"]),
    ("divide", lambda x, y: paddle.divide(x, y), dict(x=A, y=POS), lambda x, y: x / y, ["x", "y"]),
    ("pow", lambda x: paddle.pow(x, 3.0), dict(x=POS), lambda x: x ** 3, ["x"]),
    ("maximum", lambda x, y: paddle.maximum(x, y), dict(x=A, y=B), np.maximum, ["x", "y"]),
    ("exp", lambda x: paddle.exp(x), dict(x=A), np.exp, ["x"]),
    ("log", lambda x: paddle.log(x), dict(x=POS), np.log, ["x"]),
    ("sqrt", lambda x: paddle.sqrt(x), dict(x=POS), np.sqrt, ["x"]),
    ("rsqrt", lambda x: paddle.rsqrt(x), dict(x=POS), lambda x: 1 / np.sqrt(x), ["x"]),
    ("tanh", lambda x: paddle.tanh(x), dict(x=A), np.tanh, ["x"]),
    ("sigmoid", lambda x: F.sigmoid(x), dict(x=A), lambda x: 1 / (1 + np.exp(-x)), ["x"]),
    ("abs", lambda x: paddle.abs(x), dict(x=A), np.abs, ["x"]),
    ("clip", lambda x: paddle.clip(x, -0.3, 0.4), dict(x=A), lambda x: np.clip(x, -0.3, 0.4), ["x"]),
    ("scale", lambda x: paddle.scale(x, 2.0, 1.0), dict(x=A), lambda x: 2 * x + 1, ["x"]),
    ("scale_bias_first", lambda x: paddle.scale(x, 2.0, 1.0, bias_after_scale=False), dict(x=A), lambda x: 2 * (x + 1), ["x"]),
    ("sum_axis", lambda x: paddle.sum(x, axis=1, keepdim=True), dict(x=A), lambda x: x.sum(1, keepdims=True), ["x"]),
    ("mean_all", lambda x: paddle.mean(x), dict(x=A), lambda x: x.mean(), ["x"]),
    ("max_axis", lambda x: paddle.max(x, axis=0), dict(x=A), lambda x: x.max(0), ["x"]),
    ("prod", lambda x: paddle.prod(x, axis=1), dict(x=POS), lambda x: x.prod(1), ["x"]),
    ("logsumexp", lambda x: paddle.logsumexp(x, axis=1), dict(x=A), lambda x: np.log(np.exp(x).sum(1)), ["x"]),
    ("cumsum", lambda x: paddle.cumsum(x, axis=1), dict(x=A), lambda x: x.cumsum(1), ["x"]),
    ("std", lambda x: paddle.std(x, axis=1), dict(x=A), lambda x: x.std(1, ddof=1), ["x"]),
    ("var_biased", lambda x: paddle.var(x, axis=1, unbiased=False), dict(x=A), lambda x: x.var(1), ["x"]),
    ("norm_fro", lambda x: paddle.linalg.norm(x), dict(x=A), lambda x: np.sqrt((x * x).sum()), ["x"]),
    ("matmul", lambda x, y: paddle.matmul(x, y), dict(x=A, y=f32(4, 5)), lambda x, y: x @ y, ["x", "y"]),
    ("matmul_trans", lambda x, y: paddle.matmul(x, y, transpose_x=True, transpose_y=True), dict(x=f32(4, 3), y=f32(5, 4)),
     lambda x, y: x.T @ y.T, ["x", "y"]),
    ("bmm", lambda x, y: paddle.bmm(x, y), dict(x=f32(2, 3, 4), y=f32(2, 4, 2)), lambda x, y: x @ y, ["x", "y"]),
    ("dot", lambda x, y: paddle.dot(x, y), dict(x=f32(5), y=f32(5)), lambda x, y: np.dot(x, y), ["x", "y"]),
    ("transpose", lambda x: paddle.transpose(x, [1, 0, 2]), dict(x=f32(2, 3, 4)), lambda x: x.transpose(1, 0, 2), ["x"]),
    ("reshape", lambda x: paddle.reshape(x, [4, -1]), dict(x=A), lambda x: x.reshape(4, -1), ["x"]),
    ("concat", lambda x, y: paddle.concat([x, y], axis=1), dict(x=A, y=B), lambda x, y: np.concatenate([x, y], 1), ["x", "y"]),
    ("stack", lambda x, y: paddle.stack([x, y], axis=0), dict(x=A, y=B), lambda x, y: np.stack([x, y]), ["x", "y"]),
    ("split_pick", lambda x: paddle.split(x, 2, axis=1)[1], dict(x=A), lambda x: x[:, 2:], ["x"]),
    ("slice", lambda x: paddle.slice(x, [0, 1], [1, 0], [3, 2]), dict(x=A), lambda x: x[1:3, 0:2], ["x"]),
    ("gather", lambda x, index: paddle.gather(x, index), dict(x=A, index=IDX), lambda x, index: x[index], ["x"]),
    ("index_select", lambda x, index: paddle.index_select(x, index, axis=1), dict(x=A, index=IDX), lambda x, index: x[:, index], ["x"]),
    ("expand", lambda x: paddle.expand(x, [2, 3, 4]), dict(x=A), lambda x: np.broadcast_to(x, (2, 3, 4)), ["x"]),
    ("tile", lambda x: paddle.tile(x, [2, 1]), dict(x=A), lambda x: np.tile(x, (2, 1)), ["x"]),
    ("flip", lambda x: paddle.flip(x, [1]), dict(x=A), lambda x: x[:, ::-1], ["x"]),
    ("roll", lambda x: paddle.roll(x, 1, axis=1), dict(x=A), lambda x: np.roll(x, 1, 1), ["x"]),
    ("where", lambda x, y: paddle.where(x > 0, x, y), dict(x=A, y=B), lambda x, y: np.where(x > 0, x, y), ["x", "y"]),
    ("tril", lambda x: paddle.tril(x), dict(x=f32(4, 4)), np.tril, ["x"]),
    ("squeeze_unsqueeze", lambda x: paddle.unsqueeze(paddle.squeeze(x, 1), 0), dict(x=f32(3, 1, 4)), lambda x: x[:, 0][None], ["x"]),
    ("relu", lambda x: F.relu(x), dict(x=A), lambda x: np.maximum(x, 0), ["x"]),
    ("leaky_relu", lambda x: F.leaky_relu(x, 0.1), dict(x=A), lambda x: np.where(x > 0, x, 0.1 * x), ["x"]),
    ("gelu", lambda x: F.gelu(x), dict(x=A), _gelu, ["x"]),
    ("silu", lambda x: F.silu(x), dict(x=A), lambda x: x / (1 + np.exp(-x)), ["x"]),
    ("softplus", lambda x: F.softplus(x), dict(x=A), lambda x: np.log1p(np.exp(x)), ["x"]),
    ("elu", lambda x: F.elu(x, 1.0), dict(x=A), lambda x: np.where(x > 0, x, np.exp(x) - 1), ["x"]),
    ("hardswish", lambda x: F.hardswish(x), dict(x=f32(3, 4, lo=-4, hi=4)), lambda x: x * np.clip(x + 3, 0, 6) / 6, ["x"]),
    ("softmax", lambda x: F.softmax(x, axis=-1), dict(x=A), lambda x: _softmax(x, -1), ["x"]),
    ("log_softmax", lambda x: F.log_softmax(x, axis=0), dict(x=A), lambda x: np.log(_softmax(x, 0)), ["x"]),
    ("linear", lambda x, w, b: F.linear(x, w, b), dict(x=A, w=f32(4, 5), b=f32(5)), lambda x, w, b: x @ w + b, ["x", "w", "b"]),
    ("embedding", lambda ids, w: F.embedding(ids, w), dict(ids=IDX, w=f32(3, 4)), lambda ids, w: w[ids], ["w"]),
    ("layer_norm", lambda x, w, b: F.layer_norm(x, [4], w, b, 1e-5), dict(x=A, w=POS[0], b=B[0]),
     lambda x, w, b: _layer_norm_ref(x, w, b, 1e-5), ["x", "w", "b"]),
    ("conv2d", lambda x, w, b: F.conv2d(x, w, b, stride=2, padding=1), dict(x=f32(2, 3, 5, 5), w=f32(4, 3, 3, 3), b=f32(4)),
     lambda x, w, b: _conv2d_ref(x, w, b, 2, 1), ["x", "w", "b"]),
    ("avg_pool2d", lambda x: F.avg_pool2d(x, 2, 2), dict(x=f32(1, 2, 4, 4)), lambda x: _pool_ref(x, 2, 2, np.mean), ["x"]),
    ("max_pool2d", lambda x: F.max_pool2d(x, 2, 2), dict(x=f32(1, 2, 4, 4)), lambda x: _pool_ref(x, 2, 2, np.max), ["x"]),
    ("cross_entropy", lambda logits, label: F.cross_entropy(logits, label), dict(logits=f32(3, 5), label=IDX),
     _ce_ref, ["logits"]),
    ("mse_loss", lambda x, y: F.mse_loss(x, y), dict(x=A, y=B), lambda x, y: ((x - y) ** 2).mean(), ["x"]),
    ("l1_loss", lambda x, y: F.l1_loss(x, y), dict(x=A, y=B), lambda x, y: np.abs(x - y).mean(), ["x"]),
    ("bce_with_logits", lambda x, y: F.binary_cross_entropy_with_logits(x, y), dict(x=A, y=(B > 0).astype(np.float32)),
     lambda x, y: (np.maximum(x, 0) - x * y + np.log1p(np.exp(-np.abs(x)))).mean(), ["x"]),
    ("smooth_l1", lambda x, y: F.smooth_l1_loss(x, y), dict(x=A, y=B),
     lambda x, y: np.where(np.abs(x - y) < 1, 0.5 * (x - y) ** 2, np.abs(x - y) - 0.5).mean(), ["x"]),
    ("kl_div", lambda x, y: F.kl_div(x, y, reduction="sum"), dict(x=np.log(_softmax(A, -1)).astype(np.float32), y=_softmax(B, -1).astype(np.float32)),
     lambda x, y: (y * (np.log(y) - x)).sum(), ["x"]),
    ("cosine_similarity", lambda x, y: F.cosine_similarity(x, y, axis=1), dict(x=A, y=B),
     lambda x, y: (x * y).sum(1) / (np.linalg.norm(x, axis=1) * np.linalg.norm(y, axis=1)), ["x", "y"]),
    ("normalize", lambda x: F.normalize(x, axis=1), dict(x=A), lambda x: x / np.linalg.norm(x, axis=1, keepdims=True), ["x"]),
    ("pad", lambda x: F.pad(x, [1, 2], value=0.5), dict(x=f32(2, 3, 4)), lambda x: np.pad(x, ((0, 0), (0, 0), (1, 2)), constant_values=0.5), ["x"]),
    ("one_hot", lambda ids: F.one_hot(ids, 4), dict(ids=IDX), lambda ids: np.eye(4)[ids], []),
    ("argsort", lambda x: paddle.argsort(x, axis=1), dict(x=A), lambda x: np.argsort(x, 1), []),
    ("topk_values", lambda x: paddle.topk(x, 2, axis=1)[0], dict(x=A), lambda x: -np.sort(-x, 1)[:, :2], ["x"]),
    ("cast", lambda x: paddle.cast(x, "int32"), dict(x=f32(3, 4, lo=-5, hi=5)), lambda x: x.astype(np.int32), []),
    ("equal", lambda x, y: paddle.equal(x, y), dict(x=IDX, y=np.array([2, 1, 1])), lambda x, y: x == y, []),
    ("einsum", lambda x, y: paddle.einsum("ij,kj->ik", x, y), dict(x=A, y=f32(5, 4)), lambda x, y: x @ y.T, ["x", "y"]),
    ("lerp", lambda x, y: paddle.lerp(x, y, 0.3), dict(x=A, y=B), lambda x, y: x + 0.3 * (y - x), ["x", "y"]),
    ("outer", lambda x, y: paddle.outer(x, y), dict(x=f32(3), y=f32(4)), np.outer, ["x", "y"]),
    ("trace", lambda x: paddle.trace(x), dict(x=f32(4, 4)), np.trace, ["x"]),
    ("kron", lambda x, y: paddle.kron(x, y), dict(x=f32(2, 2), y=f32(2, 3)), np.kron, ["x", "y"]),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_op(case):
    name, fn, inputs, ref, grad_names = case
    np_inputs = {k: (v.astype(np.float64) if isinstance(v, np.ndarray) and v.dtype.kind == "f" else v) for k, v in inputs.items()}
    check_output(fn, inputs, ref(*np_inputs.values()), rtol=2e-5, atol=2e-6)
    if grad_names:
        check_grad(fn, inputs, grad_names)


# ------------------------------------------------------------------------------------------ second table
def _bn_train_ref(x, w, b, eps):
    m = x.mean((0, 2, 3), keepdims=True)
    v = x.var((0, 2, 3), keepdims=True)
    return (x - m) / np.sqrt(v + eps) * w.reshape(1, -1, 1, 1) + b.reshape(1, -1, 1, 1)


def _gn_ref(x, g, w, b, eps):
    n, c, h, wd = x.shape
    xg = x.reshape(n, g, -1)
    m, v = xg.mean(-1, keepdims=True), xg.var(-1, keepdims=True)
    return ((xg - m) / np.sqrt(v + eps)).reshape(x.shape) * w.reshape(1, -1, 1, 1) + b.reshape(1, -1, 1, 1)


def _conv1d_ref(x, w, pad):
    n, c, l = x.shape
    o, _, k = w.shape
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad)))
    out = np.zeros((n, o, l + 2 * pad - k + 1))
    for i in range(out.shape[-1]):
        out[:, :, i] = np.einsum("ncl,ocl->no", xp[:, :, i:i + k], w)
    return out


def _conv2d_transpose_ref(x, w, stride):
    n, c, h, wd = x.shape
    _, o, kh, kw = w.shape
    out = np.zeros((n, o, (h - 1) * stride + kh, (wd - 1) * stride + kw))
    for i in range(h):
        for j in range(wd):
            out[:, :, i * stride:i * stride + kh, j * stride:j * stride + kw] += np.einsum("nc,cokl->nokl", x[:, :, i, j], w)
    return out


def _pixel_shuffle_ref(x, r):
    n, c, h, w = x.shape
    return x.reshape(n, c // (r * r), r, r, h, w).transpose(0, 1, 4, 2, 5, 3).reshape(n, c // (r * r), h * r, w * r)


def _nearest_up2(x):
    return x.repeat(2, axis=2).repeat(2, axis=3)


def _bilinear_align_ref(x, oh, ow):
    n, c, h, w = x.shape
    ys, xs = np.linspace(0, h - 1, oh), np.linspace(0, w - 1, ow)
    y0, x0 = np.floor(ys).astype(int), np.floor(xs).astype(int)
    y1, x1 = np.minimum(y0 + 1, h - 1), np.minimum(x0 + 1, w - 1)
    wy, wx = (ys - y0)[:, None], (xs - x0)[None, :]
    g = lambda yy, xx: x[:, :, yy][:, :, :, xx]        # noqa: E731
    return g(y0, x0) * (1 - wy) * (1 - wx) + g(y0, x1) * (1 - wy) * wx + g(y1, x0) * wy * (1 - wx) + g(y1, x1) * wy * wx


def _scatter_ref(x, index, updates):
    out = x.copy()
    out[index] = updates
    return out


def _scatter_nd_add_ref(x, index, updates):
    out = x.copy()
    for i, u in zip(index, updates):
        out[tuple(i)] += u
    return out


X4 = f32(2, 4, 3, 3)
IDX2 = np.array([[1, 0, 2, 1], [0, 2, 1, 0], [2, 2, 0, 1]], dtype=np.int64)

CASES2 = [
    ("batch_norm_train", lambda x, w, b: F.batch_norm(x, paddle.zeros([4], dtype=x.dtype), paddle.ones([4], dtype=x.dtype), w, b, training=True, epsilon=1e-5),
     dict(x=X4, w=f32(4, lo=0.5, hi=1.5), b=f32(4)), lambda x, w, b: _bn_train_ref(x, w, b, 1e-5), ["x", "w", "b"]),
    ("group_norm", lambda x, w, b: F.group_norm(x, 2, 1e-5, w, b), dict(x=X4, w=f32(4, lo=0.5, hi=1.5), b=f32(4)),
     lambda x, w, b: _gn_ref(x, 2, w, b, 1e-5), ["x", "w", "b"]),
    ("instance_norm", lambda x: F.instance_norm(x, eps=1e-5), dict(x=X4),
     lambda x: (x - x.mean((2, 3), keepdims=True)) / np.sqrt(x.var((2, 3), keepdims=True) + 1e-5), ["x"]),
    ("conv1d", lambda x, w: F.conv1d(x, w, padding=1), dict(x=f32(2, 3, 6), w=f32(4, 3, 3)), lambda x, w: _conv1d_ref(x, w, 1), ["x", "w"]),
    ("conv2d_transpose", lambda x, w: F.conv2d_transpose(x, w, stride=2), dict(x=f32(1, 2, 3, 3), w=f32(2, 3, 2, 2)),
     lambda x, w: _conv2d_transpose_ref(x, w, 2), ["x", "w"]),
    ("conv2d_groups", lambda x, w: F.conv2d(x, w, groups=2), dict(x=f32(1, 4, 4, 4), w=f32(4, 2, 3, 3)),
     lambda x, w: np.concatenate([_conv2d_ref(x[:, :2], w[:2], np.zeros(2), 1, 0), _conv2d_ref(x[:, 2:], w[2:], np.zeros(2), 1, 0)], 1),
     ["x", "w"]),
    ("pixel_shuffle", lambda x: F.pixel_shuffle(x, 2), dict(x=f32(1, 8, 2, 3)), lambda x: _pixel_shuffle_ref(x, 2), ["x"]),
    ("interp_nearest", lambda x: F.interpolate(x, scale_factor=2, mode="nearest"), dict(x=f32(1, 2, 3, 3)), _nearest_up2, ["x"]),
    ("interp_bilinear_align", lambda x: F.interpolate(x, size=[5, 7], mode="bilinear", align_corners=True), dict(x=f32(1, 2, 3, 4)),
     lambda x: _bilinear_align_ref(x, 5, 7), ["x"]),
    ("adaptive_avg_pool2d", lambda x: F.adaptive_avg_pool2d(x, 1), dict(x=X4), lambda x: x.mean((2, 3), keepdims=True), ["x"]),
    ("dropout_eval", lambda x: F.dropout(x, 0.5, training=False), dict(x=A), lambda x: x, ["x"]),
    ("dropout_downscale_eval", lambda x: F.dropout(x, 0.25, training=False, mode="downscale_in_infer"), dict(x=A), lambda x: 0.75 * x, ["x"]),
    ("scatter_overwrite", lambda x, index, updates: paddle.scatter(x, index, updates), dict(x=A, index=np.array([2, 0]), updates=f32(2, 4)),
     _scatter_ref, ["x", "updates"]),
    ("scatter_nd_add", lambda x, index, updates: paddle.scatter_nd_add(x, index, updates),
     dict(x=A, index=np.array([[0, 1], [2, 3], [0, 1]]), updates=f32(3)), _scatter_nd_add_ref, ["x", "updates"]),
    ("gather_nd", lambda x, index: paddle.gather_nd(x, index), dict(x=f32(3, 4, 2), index=np.array([[0, 1], [2, 3]])),
     lambda x, index: x[index[:, 0], index[:, 1]], ["x"]),
    ("take_along_axis", lambda x, index: paddle.take_along_axis(x, index, 0), dict(x=A, index=IDX2),
     lambda x, index: np.take_along_axis(x, index, 0), ["x"]),
    ("masked_select", lambda x, y: paddle.masked_select(x, y > 0), dict(x=A, y=B), lambda x, y: x[y > 0], ["x"]),
    ("index_add", lambda x, index, v: paddle.index_add(x, index, 0, v), dict(x=A, index=np.array([0, 2]), v=f32(2, 4)),
     lambda x, index, v: _scatter_nd_add_ref(x, index[:, None], v), ["x", "v"]),
    ("cumprod", lambda x: paddle.cumprod(x, dim=1), dict(x=POS), lambda x: x.cumprod(1), ["x"]),
    ("diff", lambda x: paddle.diff(x, axis=1), dict(x=A), lambda x: np.diff(x, axis=1), ["x"]),
    ("erf", lambda x: paddle.erf(x), dict(x=A), lambda x: 2 * (_gelu(x * np.sqrt(2)) / (x * np.sqrt(2))) - 1, ["x"]),
    ("atan2", lambda x, y: paddle.atan2(x, y), dict(x=A, y=POS), np.arctan2, ["x", "y"]),
    ("log1p", lambda x: paddle.log1p(x), dict(x=POS), np.log1p, ["x"]),
    ("expm1", lambda x: paddle.expm1(x), dict(x=A), np.expm1, ["x"]),
    ("reciprocal", lambda x: paddle.reciprocal(x), dict(x=POS), lambda x: 1 / x, ["x"]),
    ("square", lambda x: paddle.square(x), dict(x=A), np.square, ["x"]),
    ("sign", lambda x: paddle.sign(x), dict(x=A), np.sign, []),
    ("floor_divide", lambda x, y: paddle.floor_divide(x, y), dict(x=np.array([7, -7, 5]), y=np.array([2, 2, -3])),
     lambda x, y: np.floor_divide(x, y), []),
    ("remainder", lambda x, y: paddle.remainder(x, y), dict(x=np.array([7, -7, 5]), y=np.array([2, 2, -3])), np.mod, []),
    ("addmm", lambda i, x, y: paddle.addmm(i, x, y, beta=0.5, alpha=2.0), dict(i=f32(3, 5), x=A, y=f32(4, 5)),
     lambda i, x, y: 0.5 * i + 2.0 * (x @ y), ["i", "x", "y"]),
    ("mv", lambda x, v: paddle.mv(x, v), dict(x=A, v=f32(4)), lambda x, v: x @ v, ["x", "v"]),
    ("dist_p2", lambda x, y: paddle.dist(x, y, 2), dict(x=A, y=B), lambda x, y: np.sqrt(((x - y) ** 2).sum()), ["x", "y"]),
    ("amax", lambda x: paddle.amax(x, axis=1), dict(x=A), lambda x: x.max(1), ["x"]),
    ("median", lambda x: paddle.median(x, axis=1), dict(x=f32(3, 5)), lambda x: np.median(x, 1), ["x"]),
    ("kthvalue", lambda x: paddle.kthvalue(x, 2, axis=1)[0], dict(x=A), lambda x: np.sort(x, 1)[:, 1], ["x"]),
    ("sort_desc", lambda x: paddle.sort(x, axis=1, descending=True), dict(x=A), lambda x: -np.sort(-x, 1), ["x"]),
    ("unbind_pick", lambda x: paddle.unbind(x, axis=1)[2], dict(x=A), lambda x: x[:, 2], ["x"]),
    ("chunk_pick", lambda x: paddle.chunk(x, 2, axis=1)[0], dict(x=A), lambda x: x[:, :2], ["x"]),
    ("moveaxis", lambda x: paddle.moveaxis(x, 0, 2), dict(x=f32(2, 3, 4)), lambda x: np.moveaxis(x, 0, 2), ["x"]),
    ("repeat_interleave", lambda x: paddle.repeat_interleave(x, 2, axis=0), dict(x=A), lambda x: x.repeat(2, 0), ["x"]),
    ("triu_diag1", lambda x: paddle.triu(x, 1), dict(x=f32(4, 4)), lambda x: np.triu(x, 1), ["x"]),
    ("diag_embed", lambda x: paddle.diag_embed(x), dict(x=f32(2, 3)), lambda x: np.stack([np.diag(r) for r in x]), ["x"]),
    ("cross", lambda x, y: paddle.cross(x, y, axis=1), dict(x=f32(2, 3), y=f32(2, 3)), lambda x, y: np.cross(x, y), ["x", "y"]),
    ("nll_loss", lambda x, label: F.nll_loss(x, label), dict(x=np.log(_softmax(f32(3, 5), -1)).astype(np.float32), label=IDX),
     lambda x, label: -x[np.arange(3), label].mean(), ["x"]),
    ("margin_ranking", lambda x, y, label: F.margin_ranking_loss(x, y, label, 0.1), dict(x=f32(5), y=f32(5), label=np.sign(f32(5)).astype(np.float32)),
     lambda x, y, label: np.maximum(0, -label * (x - y) + 0.1).mean(), ["x", "y"]),
    ("hinge_embedding", lambda x, label: F.hinge_embedding_loss(x, label, 1.0), dict(x=A, label=np.sign(B).astype(np.float32)),
     lambda x, label: np.where(label > 0, x, np.maximum(0, 1 - x)).mean(), ["x"]),
    ("label_smooth", lambda x: F.label_smooth(x, epsilon=0.1), dict(x=np.eye(4, dtype=np.float32)[IDX]), lambda x: 0.9 * x + 0.1 / 4, ["x"]),
    ("glu", lambda x: F.glu(x, axis=-1), dict(x=A), lambda x: x[:, :2] / (1 + np.exp(-x[:, 2:])), ["x"]),
    ("swish", lambda x: F.swish(x), dict(x=A), lambda x: x / (1 + np.exp(-x)), ["x"]),
    ("mish", lambda x: F.mish(x), dict(x=A), lambda x: x * np.tanh(np.log1p(np.exp(x))), ["x"]),
    ("softsign", lambda x: F.softsign(x), dict(x=A), lambda x: x / (1 + np.abs(x)), ["x"]),
    ("prelu", lambda x, w: F.prelu(x, w), dict(x=X4, w=f32(4, lo=0.1, hi=0.3)), lambda x, w: np.where(x > 0, x, w.reshape(1, -1, 1, 1) * x), ["x", "w"]),
]


@pytest.mark.parametrize("case", CASES2, ids=[c[0] for c in CASES2])
def test_op_more(case):
    name, fn, inputs, ref, grad_names = case
    np_inputs = {k: (v.astype(np.float64) if isinstance(v, np.ndarray) and v.dtype.kind == "f" else v) for k, v in inputs.items()}
    check_output(fn, inputs, ref(*np_inputs.values()), rtol=3e-5, atol=3e-6)
    if grad_names:
        check_grad(fn, inputs, grad_names)
