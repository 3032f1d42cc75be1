"""Autograd-aware operators built on the native kernels.

Dispatch rule (single code path per device, no silent fallback): a CUDA bf16 tensor always runs the
hand-written sm_100a kernel and raises if the native library is missing; CPU tensors and non-bf16
dtypes (the fp32 plumbing configuration) run the equivalent PyTorch expression.  Setting
``paddle_b200.set_kernel_policy("baseline")`` routes CUDA bf16 through library kernels instead
(cuBLAS GEMM, library attention): that is the reference-behaviour baseline used by the benchmarks.
"""
from __future__ import annotations

import math

import torch

from .._core.tensor import as_tensor
from . import native

_POLICY = "fused"  # "fused": this library's kernels; "baseline": library kernels (cuBLAS etc.)


def set_kernel_policy(policy: str):
    global _POLICY
    assert policy in ("fused", "baseline")
    _POLICY = policy


def get_kernel_policy() -> str:
    return _POLICY


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and _POLICY == "fused"


# ------------------------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
    """y = x @ W (+ b) with W stored ``[in, out]`` (Paddle layout, python/paddle/nn/functional/common.py:2238).

    Backward computes dX with a K-major x K-major GEMM and dW with an MN-major x MN-major GEMM whose
    epilogue adds straight into ``weight.main_grad`` when the parameter carries one (the reference's
    fused_linear_param_grad_add), so no bf16 dW tensor is ever materialised."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if bias is not None and bias.dtype == torch.bfloat16 and bias.is_contiguous() and weight.shape[1] % 8 == 0:
            y = native.gemm_epilogue(x2, weight, bias)          # bias added in the GEMM epilogue
        else:
            y = native.gemm(x2, weight)
            if bias is not None:
                y = y + bias
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        ctx.weight_ref = weight
        return y.view(*x.shape[:-1], weight.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = native.gemm(dy2, weight, trans_b=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.weight_ref, "main_grad", None)
            if mg is not None:
                native.gemm(x2, dy2, trans_a=True, out=mg, accumulate=True)
                dw = None
                hook = getattr(ctx.weight_ref, "_main_grad_ready_hook", None)
                if hook is not None:
                    hook(ctx.weight_ref)
            else:
                dw = native.gemm(x2, dy2, trans_a=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db


class WeightGradStore:
    """Deferred weight gradients for zero-bubble pipeline schedules.  While ``split`` is set, ``linear`` records a
    node whose backward can leave out the weight gradient; while ``enabled`` is set as well, that backward produces
    only the input gradient and queues the weight (and bias) gradient as a closure.  ``flush()`` runs what has been
    queued, ``pop()`` hands that batch to the caller so a schedule can run it in a later "W" step.
    The reference splits matmul_grad into two matmul ops for the same purpose
    (python/paddle/distributed/passes/pipeline_scheduler_pass/pipeline_zero_bubble.py:38-60)."""
    split = False
    enabled = False
    _queue: list = []

    @classmethod
    def put(cls, fn):
        cls._queue.append(fn)

    @classmethod
    def pop(cls):
        batch, cls._queue = cls._queue, []
        return batch

    @classmethod
    def flush(cls):
        for fn in cls.pop():
            fn()

    @staticmethod
    def run(batch):
        for fn in batch:
            fn()


class _SplitLinearFn(torch.autograd.Function):
    """Linear whose backward returns dX at once and leaves dW / db to ``WeightGradStore``."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        use_native = _native(x) and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and weight.shape[1] % 8 == 0
        if use_native and not x2.is_contiguous():
            x2 = x2.contiguous()
        y = native.gemm(x2, weight) if use_native else x2 @ weight
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(x2, weight)
        ctx.use_native, ctx.x_shape = use_native, x.shape
        ctx.weight_ref, ctx.bias_ref = weight, bias
        return y.view(*x.shape[:-1], weight.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if ctx.use_native and not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = (native.gemm(dy2, weight, trans_b=True) if ctx.use_native else dy2 @ weight.t()).view(ctx.x_shape)
        w, b, use_native = ctx.weight_ref, ctx.bias_ref, ctx.use_native
        need_w, need_b = ctx.needs_input_grad[1], b is not None and ctx.needs_input_grad[2]

        def weight_grad():
            with torch.no_grad():
                if need_w:
                    mg = getattr(w, "main_grad", None)
                    if mg is not None and use_native:
                        native.gemm(x2, dy2, trans_a=True, out=mg, accumulate=True)
                    else:
                        dw = native.gemm(x2, dy2, trans_a=True) if use_native else x2.t() @ dy2
                        if mg is not None:
                            mg.add_(dw)
                        elif w.grad is None:
                            w.grad = dw
                        else:
                            w.grad.add_(dw)
                    hook = getattr(w, "_main_grad_ready_hook", None)
                    if mg is not None and hook is not None:
                        hook(w)
                if need_b:
                    db = dy2.sum(0).to(b.dtype)
                    if b.grad is None:
                        b.grad = db
                    else:
                        b.grad.add_(db)

        if WeightGradStore.enabled:
            WeightGradStore.put(weight_grad)
        else:
            weight_grad()
        return dx, None, None


def linear(x, weight, bias=None):
    if WeightGradStore.split and x.dim() >= 2 and weight.dim() == 2 and torch.is_grad_enabled():
        return as_tensor(_SplitLinearFn.apply(x, weight, bias))
    if _native(x) and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and weight.shape[1] % 8 == 0:
        return as_tensor(_LinearFn.apply(x, weight, bias))
    y = torch.matmul(x, weight)
    return y if bias is None else y + bias


class _MatmulFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, ta, tb):
        ctx.save_for_backward(a, b)
        ctx.ta, ctx.tb = ta, tb
        return native.gemm(a, b, ta, tb)

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        ta, tb = ctx.ta, ctx.tb
        dc = dc.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            # C = op(A) op(B):  d op(A) = dC op(B)^T ; stored-layout gradient transposes again if ta
            da = native.gemm(b, dc, tb, True) if ta else native.gemm(dc, b, False, not tb)
        if ctx.needs_input_grad[1]:
            db = native.gemm(dc, a, True, ta) if tb else native.gemm(a, dc, not ta, False)
        return da, db, None, None


def matmul(x, y, transpose_x=False, transpose_y=False):
    if (_native(x) and y.dtype == torch.bfloat16 and x.dim() == 2 and y.dim() == 2 and x.is_contiguous()
            and y.is_contiguous() and all(s % 8 == 0 for s in (*x.shape, *y.shape))):
        return as_tensor(_MatmulFn.apply(x, y, bool(transpose_x), bool(transpose_y)))
    if _native(x) and y.dim() == 2 and x.dim() > 2 and not transpose_x and not transpose_y \
            and y.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and y.shape[1] % 8 == 0 and y.is_contiguous():
        return linear(x, y)
    a = x.mT if transpose_x and x.dim() > 1 else x
    b = y.mT if transpose_y and y.dim() > 1 else y
    return torch.matmul(a, b)


# ------------------------------------------------------------------------------------------- rms norm
class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual):
        y, inv, res_out = native.rms_norm_fwd(x, w, eps, residual=residual, want_residual_out=residual is not None)
        src = res_out if residual is not None else x
        ctx.save_for_backward(src, w, inv)
        ctx.has_res = residual is not None
        ctx.w_ref = w
        return y, res_out

    @staticmethod
    def backward(ctx, dy, dres):
        src, w, inv = ctx.saved_tensors
        mg = getattr(ctx.w_ref, "main_grad", None)
        dx, dw = native.rms_norm_bwd(dy.contiguous(), src, w, inv,
                                     dx_add=dres.contiguous() if (ctx.has_res and dres is not None) else None,
                                     dw_out=mg)
        if mg is not None:
            dw_ret = None
            hook = getattr(ctx.w_ref, "_main_grad_ready_hook", None)
            if hook is not None:
                hook(ctx.w_ref)
        else:
            dw_ret = dw.to(w.dtype)
        return dx, dw_ret, None, (dx if ctx.has_res else None)


def rms_norm(x, weight, eps=1e-6, residual=None):
    """Returns ``y`` (and the pre-norm sum when ``residual`` is given)."""
    if _native(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        xc = x if x.is_contiguous() else x.contiguous()
        rc = None if residual is None else (residual if residual.is_contiguous() else residual.contiguous())
        y, res_out = _RmsNormFn.apply(xc, weight, eps, rc)
        return (as_tensor(y), as_tensor(res_out)) if residual is not None else as_tensor(y)
    s = x if residual is None else x + residual
    sf = s.float()
    y = (sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)
    return (y, s) if residual is not None else y


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        y, mean, rstd = native.layer_norm_fwd(x, w, b, eps)
        ctx.save_for_backward(x, w, mean, rstd)
        ctx.has_bias = b is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        dx, dw, db = native.layer_norm_bwd(dy.contiguous(), x, w, mean, rstd)
        return dx, dw.to(w.dtype), (db.to(w.dtype) if ctx.has_bias else None), None


def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    H = x.shape[-1]
    if (_native(x) and weight is not None and H % 8 == 0 and H <= 8192
            and (isinstance(normalized_shape, int) or len(normalized_shape) == 1)):
        if bias is not None and bias.dtype != weight.dtype:
            bias = bias.to(weight.dtype)
        return as_tensor(_LayerNormFn.apply(x.contiguous(), weight, bias, eps))
    ns = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
    return torch.nn.functional.layer_norm(x, ns, weight, bias, eps)


# ------------------------------------------------------------------------------------------- rope
_rope_cache = {}


def rope_tables(seq_len: int, dim: int, base: float, device, half_style: bool = True):
    """fp32 ``[seq_len, dim]`` cos / sin tables in the pairing convention of the kernel."""
    key = (seq_len, dim, float(base), str(device), half_style)
    t = _rope_cache.get(key)
    if t is None:
        inv = 1.0 / (base ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
        ang = torch.arange(seq_len, device=device, dtype=torch.float32)[:, None] * inv[None]
        if half_style:
            cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
        else:
            cos, sin = ang.cos().repeat_interleave(2, -1), ang.sin().repeat_interleave(2, -1)
        t = (cos.contiguous(), sin.contiguous())
        _rope_cache[key] = t
    return t


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, position_ids, half_style):
        ctx.save_for_backward(cos, sin, position_ids)
        ctx.half_style = half_style
        return native.rope(x, cos, sin, position_ids, half_style=half_style)

    @staticmethod
    def backward(ctx, dy):
        cos, sin, pid = ctx.saved_tensors
        if not (dy.stride(-1) == 1 and dy.stride(-2) == dy.shape[-1]):
            dy = dy.contiguous()
        return native.rope(dy, cos, sin, pid, half_style=ctx.half_style, backward=True), None, None, None, None


def _rope_torch(x, cos, sin, position_ids, half_style):
    D = x.shape[-1]
    if position_ids is not None:
        c, s = cos[position_ids][:, :, None, :], sin[position_ids][:, :, None, :]
    else:
        S = x.shape[-3]
        c, s = cos[:S][None, :, None, :], sin[:S][None, :, None, :]
    xf = x.float()
    if half_style:
        rot = torch.cat([-xf[..., D // 2:], xf[..., :D // 2]], -1)
    else:
        rot = torch.stack([-xf[..., 1::2], xf[..., 0::2]], -1).reshape(xf.shape)
    return (xf * c + rot * s).to(x.dtype)


def rope(x, cos, sin, position_ids=None, half_style=True):
    """Rotary embedding on ``[batch, seq, heads, dim]``; cos/sin are fp32 ``[max_pos, dim]``."""
    if _native(x) and x.shape[-1] % 16 == 0 and x.dim() >= 3:
        ok = x.stride(-1) == 1 and x.stride(-2) == x.shape[-1] and all(
            x.stride(i) == x.stride(i + 1) * x.shape[i + 1] for i in range(x.dim() - 3))
        if not ok:
            x = x.contiguous()
        return as_tensor(_RopeFn.apply(x, cos, sin, position_ids, half_style))
    return _rope_torch(x, cos, sin, position_ids, half_style)


# ------------------------------------------------------------------------------------------- swiglu
class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y):
        ctx.save_for_backward(x, y)
        return native.swiglu_fwd(x, y)

    @staticmethod
    def backward(ctx, dout):
        x, y = ctx.saved_tensors
        dx, dy = native.swiglu_bwd(x, y, dout)
        return dx, dy


def swiglu(x, y=None):
    """``silu(x) * y``; with ``y=None`` the last axis of ``x`` is split in halves
    (python/paddle/incubate/nn/functional/swiglu.py:58)."""
    F = x.shape[-1] if y is not None else x.shape[-1] // 2
    if _native(x) and F % 8 == 0:
        x = x.contiguous()
        return as_tensor(_SwigluFn.apply(x, None if y is None else y.contiguous()))
    if y is None:
        x, y = x.chunk(2, -1)
    return torch.nn.functional.silu(x) * y


# ------------------------------------------------------------------------------------------- CE
class _SoftmaxCEFn(torch.autograd.Function):
    """Hard-label softmax cross entropy per row; logits [T, V].  The gradient overwrites nothing:
    the logits tensor is kept and read once more in backward."""

    @staticmethod
    def forward(ctx, logits, labels, ignore_index):
        mx, sm, tg, loss = native.ce_stats(logits, labels, 0, ignore_index)
        ctx.save_for_backward(logits, labels, mx + sm.log())
        ctx.ignore_index = ignore_index
        return loss

    @staticmethod
    def backward(ctx, dloss):
        logits, labels, lse = ctx.saved_tensors
        return native.ce_bwd(logits, labels, lse, dloss.contiguous(), 0, ctx.ignore_index), None, None


def softmax_cross_entropy(logits, labels, ignore_index=-100):
    """Per-token loss (fp32) for hard labels: logits ``[..., V]``, labels ``[...]``."""
    V = logits.shape[-1]
    lead = logits.shape[:-1]
    if logits.is_cuda and _POLICY == "fused" and logits.dtype in (torch.bfloat16, torch.float32) \
            and V % (8 if logits.dtype == torch.bfloat16 else 4) == 0:
        l2 = logits.reshape(-1, V)
        if not l2.is_contiguous():
            l2 = l2.contiguous()
        return as_tensor(_SoftmaxCEFn.apply(l2, labels.reshape(-1), ignore_index)).view(lead)
    l2 = logits.reshape(-1, V)
    if l2.dtype != torch.float64:                       # low precision is promoted to fp32, double stays double
        l2 = l2.float()
    return torch.nn.functional.cross_entropy(l2, labels.reshape(-1).long(), reduction="none",
                                             ignore_index=ignore_index).view(lead)


# ------------------------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, vocab_start, padding_idx):
        ctx.save_for_backward(ids)
        ctx.table_ref = table
        ctx.vocab_start, ctx.padding_idx = vocab_start, padding_idx
        return native.embedding_fwd(ids, table, vocab_start)

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        table = ctx.table_ref
        mg = getattr(table, "main_grad", None)
        if mg is not None:
            native.embedding_bwd(ids, dout, mg, ctx.vocab_start, ctx.padding_idx)
            hook = getattr(table, "_main_grad_ready_hook", None)
            if hook is not None:
                hook(table)
            return None, None, None, None
        dt = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        native.embedding_bwd(ids, dout, dt, ctx.vocab_start, ctx.padding_idx)
        return None, dt.to(table.dtype), None, None


def embedding(ids, table, padding_idx=None, vocab_start=0, sharded=False):
    if _native(table) and table.shape[1] % 8 == 0:
        return as_tensor(_EmbeddingFn.apply(ids, table, vocab_start, -1 if padding_idx is None else padding_idx))
    if vocab_start == 0 and not sharded:
        return torch.nn.functional.embedding(ids, table, padding_idx=padding_idx)
    local = ids - vocab_start
    ok = (local >= 0) & (local < table.shape[0])
    out = torch.nn.functional.embedding(local.clamp(0, table.shape[0] - 1), table)
    return out * ok.unsqueeze(-1).to(out.dtype)


# ------------------------------------------------------------------------------------------- dropout
def _next_philox(n):
    """(seed, offset) of the current CUDA generator for a dropout over ``n`` elements; advances the generator, so the
    saved / restored generator state (RNG tracker, recompute) reproduces the same masks."""
    gen = torch.cuda.default_generators[torch.cuda.current_device()]
    seed, offset = gen.initial_seed(), gen.get_offset()
    gen.set_offset(offset + native.dropout_offset_step(n))
    return seed, offset


class _DropoutAddFn(torch.autograd.Function):
    """out = dropout(x) [+ y]; backward regenerates the keep decisions from (seed, offset) - no mask is stored
    (paddle/phi/kernels/fusion/gpu/fused_dropout_add_grad_kernel.cu)."""

    @staticmethod
    def forward(ctx, x, y, p, upscale, seed, offset):
        ctx.meta = (p, upscale, seed, offset, y is not None)
        return native.dropout_add(x, y, p, upscale, seed, offset)

    @staticmethod
    def backward(ctx, dout):
        p, upscale, seed, offset, has_y = ctx.meta
        dout = dout.contiguous()
        dx = native.dropout_add(dout, None, p, upscale, seed, offset) if ctx.needs_input_grad[0] else None
        return dx, (dout if has_y else None), None, None, None, None


def dropout_add_supported(x, y=None):
    return (_native_any(x) and x.dtype in (torch.bfloat16, torch.float32) and x.is_contiguous()
            and (y is None or (y.shape == x.shape and y.dtype == x.dtype and y.is_contiguous()))
            and not torch.cuda.is_current_stream_capturing())


def _native_any(x):
    return isinstance(x, torch.Tensor) and x.is_cuda and _POLICY == "fused"


def dropout_add(x, y, p, upscale=True, seed_offset=None):
    """``dropout(x) + y`` (``y`` may be None) in one kernel; returns ``(out, (seed, offset))``."""
    seed, offset = seed_offset if seed_offset is not None else _next_philox(x.numel())
    return as_tensor(_DropoutAddFn.apply(x, y, float(p), bool(upscale), int(seed), int(offset))), (seed, offset)


# ------------------------------------------------------------------------------------------- attention
def _sdpa_reference(q, k, v, causal, scale):
    # [b, s, h, d] -> [b, h, s, d]; GQA by head repetition
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if kh.shape[1] != qh.shape[1]:
        rep = qh.shape[1] // kh.shape[1]
        kh, vh = kh.repeat_interleave(rep, 1), vh.repeat_interleave(rep, 1)
    o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=scale)
    return o.transpose(1, 2)


def flash_attention(q, k, v, causal=False, scale=None):
    """softmax(q k^T * scale + causal mask) v on ``[batch, seq, heads, head_dim]`` tensors
    (python/paddle/nn/functional/flash_attention.py:358).  Returns the output only."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if _native(q):
        from . import attention
        if attention.supported(q, k, v):
            return as_tensor(attention.flash_attn_func(q, k, v, causal, scale))
    return _sdpa_reference(q, k, v, causal, scale)
