"""``paddle.nn.quant``: weight-only quantised linears (python/paddle/nn/quant/quantized_linear.py) and ``Stub``
(python/paddle/nn/quant/stub.py).

``weight_quantize`` returns the weight transposed to ``[out, in]`` in int8 (int4 packs two values per byte along the
input dimension) with per-output-channel or per-group scales; ``weight_only_linear`` dequantises into the
activation dtype and runs the GEMM on the tensor cores, so weight traffic from HBM is halved or quartered for the
memory-bound small-batch case."""
from __future__ import annotations

import torch

from ..._core.tensor import as_tensor
from ..layer.layers import Layer


def _p(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


def _check_algo(algo):
    if algo not in ("weight_only_int8", "weight_only_int4", "llm.int8"):
        raise ValueError(f"algo must be one of weight_only_int8 / weight_only_int4 / llm.int8, got {algo}")


def weight_quantize(x, algo="weight_only_int8", arch=None, group_size=-1):
    """``x``: [in, out] float weight.  Returns ``(quantised [out, in] int8 (int4: [out, in / 2]), scale)`` with
    ``scale`` [out] (per channel) or [in / group_size, out] (grouped)."""
    _check_algo(algo)
    if group_size not in (-1, 64, 128):
        raise ValueError("group_size only supports -1 (per channel), 64 or 128")
    w = _p(x).float()
    qmax = 7.0 if algo == "weight_only_int4" else 127.0
    K, N = w.shape
    if group_size == -1:
        scale = w.abs().amax(0).clamp_min(1e-8) / qmax                 # [N]
        q = torch.round(w / scale).clamp(-qmax, qmax)
    else:
        g = w.reshape(K // group_size, group_size, N)
        scale = g.abs().amax(1).clamp_min(1e-8) / qmax                 # [K/g, N]
        q = torch.round(g / scale[:, None]).clamp(-qmax, qmax).reshape(K, N)
    q = q.t().contiguous().to(torch.int8)                              # [N, K]
    if algo == "weight_only_int4":
        lo, hi = q[:, 0::2] & 0xF, q[:, 1::2] & 0xF
        q = (lo | (hi << 4)).to(torch.int8)
    return as_tensor(q), as_tensor(scale.to(_p(x).dtype if _p(x).dtype != torch.float32 else torch.float32))


def _unpack(weight, weight_dtype):
    q = _p(weight)
    if weight_dtype == "int4":
        lo = (q << 4).to(torch.int8) >> 4                              # sign-extend the low nibble
        hi = q >> 4
        q = torch.stack([lo, hi], -1).reshape(q.shape[0], -1)
    return q


def weight_dequantize(x, scale, algo="weight_only_int8", out_dtype="float16", group_size=-1):
    """Inverse of :func:`weight_quantize`: returns the ``[in, out]`` weight in ``out_dtype``."""
    from ..._core import dtype as _dt
    _check_algo(algo)
    q = _unpack(x, "int4" if algo == "weight_only_int4" else "int8").float()        # [N, K]
    s = _p(scale).float()
    if group_size == -1:
        w = q * s[:, None]
    else:
        N, K = q.shape
        w = (q.reshape(N, K // group_size, group_size) * s.t()[:, :, None]).reshape(N, K)
    return as_tensor(w.t().contiguous().to(_dt.to_torch(out_dtype)))


def weight_only_linear(x, weight, bias=None, weight_scale=None, weight_dtype="int8", arch=None, group_size=-1):
    xa = _p(x)
    q = _unpack(weight, weight_dtype)                                   # [N, K] int8
    s = _p(weight_scale)
    if group_size == -1:
        # scale per output channel commutes with the GEMM: y = (x @ q^T) * s
        y = torch.matmul(xa, q.to(xa.dtype).t()) * s.to(xa.dtype)
    else:
        N, K = q.shape
        w = (q.reshape(N, K // group_size, group_size).to(xa.dtype) * s.t().to(xa.dtype)[:, :, None]).reshape(N, K)
        y = torch.matmul(xa, w.t())
    if bias is not None:
        y = y + _p(bias)
    return as_tensor(y)


def llm_int8_linear(x, weight, bias=None, weight_scale=None, threshold=6.0):
    """LLM.int8(): activation columns with an outlier (|x| > threshold) go through the floating-point path, the rest
    are quantised per row to int8 and multiplied with the int8 weight."""
    xa = _p(x)
    q = _p(weight)                                                      # [N, K] int8
    s = _p(weight_scale).float()
    x2 = xa.reshape(-1, xa.shape[-1]).float()
    outlier = (x2.abs() > threshold).any(0)                             # [K]
    w_f = q.float() * s[:, None]
    y = x2[:, outlier] @ w_f[:, outlier].t()
    xn = x2[:, ~outlier]
    if xn.shape[1]:
        xs = xn.abs().amax(1, keepdim=True).clamp_min(1e-8) / 127.0
        xq = torch.round(xn / xs).clamp(-127, 127)
        y = y + (xq @ q[:, ~outlier].float().t()) * xs * s
    y = y.reshape(*xa.shape[:-1], -1).to(xa.dtype)
    if bias is not None:
        y = y + _p(bias)
    return as_tensor(y)


class Stub(Layer):
    """Placeholder that a quantisation pass replaces with the observer / quanter configured for it."""

    def __init__(self, observer=None):
        super().__init__()
        self._observer = observer

    def forward(self, input):
        return input
