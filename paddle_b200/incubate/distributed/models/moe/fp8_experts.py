"""SwiGLU experts of one rank as two grouped GEMMs with block-scaled fp8 operands, trainable.

The reference runs every expert as its own pair of ``Linear`` layers on that expert's slice of the routed tokens
(python/paddle/incubate/distributed/models/moe/moe_layer.py:419-440) and has fp8 GEMMs only per tensor
(paddle/phi/kernels/fusion/fp8_gemm/fp8_gemm_with_cublasLt/cublaslt_gemm.h:68).  Here the experts' weights are
stacked (``[E, K, N]``) and all experts run in one launch per GEMM:

* forward   ``Y = grouped(Xq, Wq)``          X quantised per 1 x 128 block, W per 128 x 128 block (e4m3, fp32 scales)
* dgrad     ``dX = grouped(dYq, (W^T)q)``    the same kernel on a byte-transposed copy of the e4m3 weights
* wgrad     ``dW[e] = X_e^T dY_e``           bf16 operands on the plain tcgen05 GEMM, fp32 accumulation into
                                            ``main_grad`` when the parameter carries one

Quantised weights are cached between optimizer steps (micro-batches of one step reuse them) and keyed on the
parameter's version counter, which this library's optimizers advance; ``weights_updated()`` drops them by hand for
code that writes the parameters through other means.  Off the GPU the same module computes the
per-expert products with plain matmuls, so routing and parity tests run anywhere."""
from __future__ import annotations

import torch

from ..... import nn
from ....._core.tensor import as_tensor
from .....nn.initializer import Normal
from .....ops import functional as K
from .....ops import native


def _on_gpu(x, w):
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[1] % 128 == 0 and w.shape[2] % 128 == 0)


class _QuantCache:
    """e4m3 copies of a stacked weight for the forward (``W``) and the input-gradient (``W^T``) GEMMs."""

    def __init__(self):
        self.key = None
        self.fwd = self.bwd = None

    def get(self, w, transposed):
        key = (w.data_ptr(), w._version)
        if key != self.key:
            self.key, self.fwd, self.bwd = key, None, None
        if self.fwd is None:
            self.fwd = native.fp8_quant_weight(w.detach().contiguous())
        if transposed:
            if self.bwd is None:
                # 128 x 128 blocks of W and of W^T hold the same values, so the operand of the input-gradient GEMM
                # is the transposed e4m3 copy with the transposed scale grid: a byte transpose, no second
                # quantisation pass over the bf16 weights
                q, s = self.fwd
                self.bwd = (q.view(torch.uint8).transpose(1, 2).contiguous().view(torch.float8_e4m3fn),
                            s.transpose(1, 2).contiguous())
            return self.bwd
        return self.fwd

    def clear(self):
        self.key = self.fwd = self.bwd = None


class _GroupedLinearFP8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, offsets, counts, cache):
        xq, xs = native.fp8_quant_1x128(x.contiguous())
        wq, ws = cache.get(w, False)
        y = native.grouped_gemm_fp8(xq, xs, wq, ws, offsets)
        ctx.save_for_backward(x, w, offsets)
        ctx.counts, ctx.cache, ctx.w_ref = counts, cache, w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, offsets = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dq, ds = native.fp8_quant_1x128(dy)
            wq, ws = ctx.cache.get(w, True)
            dx = native.grouped_gemm_fp8(dq, ds, wq, ws, offsets)
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is None:
                dw = torch.zeros_like(w)
            start = 0
            for e, n in enumerate(ctx.counts):
                if n:
                    xe, de = x[start:start + n], dy[start:start + n]
                    if mg is not None:
                        native.gemm(xe, de, trans_a=True, out=mg[e], accumulate=True)
                    else:
                        native.gemm(xe, de, trans_a=True, out=dw[e])
                start += n
        return dx, dw, None, None, None


def _grouped_linear_plain(x, w, counts):
    outs, start = [], 0
    for e, n in enumerate(counts):
        if n:
            outs.append(x[start:start + n] @ w[e])
        start += n
    return torch.cat(outs, 0) if outs else x.new_zeros((0, w.shape[2]))


def grouped_linear(x, w, counts, cache=None, offsets=None):
    """Rows of ``x`` are sorted by expert, ``counts[e]`` of them belong to expert ``e``; returns ``[M, N]`` with row
    ``i`` of expert ``e`` equal to ``x[i] @ w[e]``."""
    counts = [int(c) for c in counts]
    if x.shape[0] == 0 or not _on_gpu(x, w):
        return as_tensor(_grouped_linear_plain(x, w, counts))
    if offsets is None:
        offsets = torch.tensor([0] + counts, dtype=torch.int32).cumsum(0).to(torch.int32).to(x.device, non_blocking=True)
    return as_tensor(_GroupedLinearFP8.apply(x, w, offsets, counts, cache if cache is not None else _QuantCache()))


class FP8GroupedExperts(nn.Layer):
    """``num_experts`` SwiGLU feed-forward experts with stacked weights; ``forward(x, counts)`` takes the routed tokens
    ordered by expert.  ``MoELayer`` accepts an instance in place of a list of expert layers."""
    grouped = True

    def __init__(self, num_experts, hidden_size, intermediate_size, initializer_range=0.02):
        super().__init__()
        self.num_experts, self.hidden_size, self.intermediate_size = num_experts, hidden_size, intermediate_size
        init = nn.ParamAttr(initializer=Normal(0.0, initializer_range))
        self.gate_up_weight = self.create_parameter([num_experts, hidden_size, 2 * intermediate_size], attr=init)
        self.down_weight = self.create_parameter([num_experts, intermediate_size, hidden_size], attr=init)
        self._cache = (_QuantCache(), _QuantCache())

    def __len__(self):
        return self.num_experts

    def weights_updated(self):
        """Drop the cached e4m3 weights (call after an optimizer step that wrote the parameters in place)."""
        for c in self._cache:
            c.clear()

    def forward(self, x, counts):
        counts = [int(c) for c in (counts.tolist() if hasattr(counts, "tolist") else counts)]
        offsets = None
        if x.is_cuda:
            offsets = torch.tensor([0] + counts, dtype=torch.int32).cumsum(0).to(torch.int32).to(x.device, non_blocking=True)
        h = grouped_linear(x, self.gate_up_weight, counts, self._cache[0], offsets)
        a = K.swiglu(h)
        return grouped_linear(a, self.down_weight, counts, self._cache[1], offsets)
