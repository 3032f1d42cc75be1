"""Flash attention on the sm_100a kernels: autograd wrapper and shape gate."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import c_float, c_int, c_int64, check, ptr, stream
from . import native


def supported(q, k, v) -> bool:
    return (q.dim() == 4 and q.shape[-1] == 128 and k.shape[-1] == 128 and v.shape[-1] == 128
            and q.dtype == k.dtype == v.dtype == torch.bfloat16 and q.shape[2] % k.shape[2] == 0
            and k.shape[2] == v.shape[2] and k.shape[1] == v.shape[1])


def _view_ok(t):
    # [B, S, H, 128] with dense heads; token / batch strides free but 16-byte aligned
    return (t.stride(3) == 1 and t.stride(2) == 128 and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


def fwd(q, k, v, causal, scale):
    q, k, v = (t if _view_ok(t) else t.contiguous() for t in (q, k, v))
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    o = torch.empty((B, Sq, Hq, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    rc = _lib.kernels().pd_flash_attn_fwd(
        ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), c_int(B), c_int(Sq), c_int(Sk), c_int(Hq), c_int(Hkv),
        c_int64(q.stride(1)), c_int64(q.stride(0)), c_int64(k.stride(1)), c_int64(k.stride(0)),
        c_int64(v.stride(1)), c_int64(v.stride(0)), c_int64(o.stride(1)), c_int64(o.stride(0)),
        c_float(scale), c_int(1 if causal else 0), ptr(_lib.status_buffer(q.device)), stream())
    check(rc, "pd_flash_attn_fwd")
    native._count()
    return o, lse


def bwd(do, q, k, v, o, lse, causal, scale):
    k_ = _lib.kernels()
    if not hasattr(k_, "pd_flash_attn_bwd"):
        raise _lib.NativeLibraryError("pd_flash_attn_bwd is missing from libpd_kernels.so")
    q, k, v, o, do = (t if _view_ok(t) else t.contiguous() for t in (q, k, v, o, do))
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    dq = torch.empty((B, Sq, Hq, D), dtype=torch.bfloat16, device=q.device)
    dk = torch.empty((B, Sk, Hkv, D), dtype=torch.bfloat16, device=q.device)
    dv = torch.empty((B, Sk, Hkv, D), dtype=torch.bfloat16, device=q.device)
    dq_acc = torch.zeros((B, Sq, Hq, D), dtype=torch.float32, device=q.device)
    delta = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    g = Hq // Hkv
    dkv_acc = torch.zeros((2, B, Sk, Hkv, D), dtype=torch.float32, device=q.device) if g > 1 else None
    rc = k_.pd_flash_attn_bwd(
        ptr(do), ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), ptr(delta), ptr(dq_acc), ptr(dkv_acc), ptr(dq), ptr(dk),
        ptr(dv), c_int(B), c_int(Sq), c_int(Sk), c_int(Hq), c_int(Hkv),
        c_int64(q.stride(1)), c_int64(q.stride(0)), c_int64(k.stride(1)), c_int64(k.stride(0)),
        c_int64(v.stride(1)), c_int64(v.stride(0)), c_int64(o.stride(1)), c_int64(o.stride(0)),
        c_int64(do.stride(1)), c_int64(do.stride(0)),
        c_float(scale), c_int(1 if causal else 0), ptr(_lib.status_buffer(q.device)), stream())
    check(rc, "pd_flash_attn_bwd")
    native._count(3)
    return dq, dk, dv


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        o, lse = fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale = causal, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = bwd(do, q, k, v, o, lse, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


def flash_attn_func(q, k, v, causal, scale):
    return _FlashAttnFn.apply(q, k, v, bool(causal), float(scale))
