"""Flash attention on the sm_100a kernels: raw launches, autograd wrappers and the fused
rotary-embedding + attention operator that works in place on a packed qkv projection."""
from __future__ import annotations

import torch

from . import _lib, native
from ._lib import c_float, c_int, c_int64, check, ptr, stream


def supported(q, k, v) -> bool:
    return (q.dim() == 4 and q.shape[-1] == 128 and k.shape[-1] == 128 and v.shape[-1] == 128
            and q.dtype == k.dtype == v.dtype == torch.bfloat16 and q.shape[2] % k.shape[2] == 0
            and k.shape[2] == v.shape[2] and k.shape[1] == v.shape[1])


def _view_ok(t):
    # [B, S, H, 128] with dense heads; token / batch strides free but 16-byte aligned
    return (t.stride(3) == 1 and t.stride(2) == 128 and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


INT_MAX = 2 ** 31 - 1


def normalize_flashmask(startend_row_indices, causal, seq_q):
    """Paddle's ``startend_row_indices`` ``[B, Hm, Sk, 1 | 2 | 4]`` (flashmask_attention,
    python/paddle/nn/functional/flash_attention.py:1343-1362) as the kernels' uniform form: int32 ``[B, Hm, Sk, 4]`` of
    ``{lts, lte, uts, ute}`` - query row r does not see the column iff ``lts <= r < lte`` or ``uts <= r < ute`` - and
    the per-128-column summary ``[B, Hm, ceil(Sk / 128), 4]`` of ``{max lts, min lte, max uts, min ute}``."""
    idx = startend_row_indices.to(torch.int32)
    nb = idx.shape[-1]
    lts = idx[..., 0]
    zeros = torch.zeros_like(lts)
    big = torch.full_like(lts, INT_MAX)
    if causal:
        assert nb in (1, 2), "causal flashmask takes [lts] or [lts, lte]"
        parts = (lts, idx[..., 1] if nb == 2 else big, zeros, zeros)
    else:
        assert nb in (2, 4), "non-causal flashmask takes [lts, ute] or [lts, lte, uts, ute]"
        parts = (lts, big, zeros, idx[..., 1]) if nb == 2 else (lts, idx[..., 1], idx[..., 2], idx[..., 3])
    bounds = torch.stack(parts, -1).contiguous()
    B, Hm, Sk, _ = bounds.shape
    tiles = (Sk + 127) // 128
    pad = tiles * 128 - Sk
    neutral = torch.tensor([-INT_MAX, INT_MAX, -INT_MAX, INT_MAX], dtype=torch.int32, device=bounds.device)
    padded = torch.cat([bounds, neutral.expand(B, Hm, pad, 4)], 2) if pad else bounds
    t = padded.view(B, Hm, tiles, 128, 4)
    tile_bounds = torch.stack([t[..., 0].amax(-1), t[..., 1].amin(-1), t[..., 2].amax(-1), t[..., 3].amin(-1)], -1)
    return bounds, tile_bounds.contiguous()


def fwd(q, k, v, causal, scale, mask=None):
    """``mask``: optional ``(bounds, tile_bounds)`` from :func:`normalize_flashmask`."""
    q, k, v = (t if _view_ok(t) else t.contiguous() for t in (q, k, v))
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    o = torch.empty((B, Sq, Hq, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    rc = _lib.kernels().pd_flash_attn_fwd(
        ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), c_int(B), c_int(Sq), c_int(Sk), c_int(Hq), c_int(Hkv),
        c_int64(q.stride(1)), c_int64(q.stride(0)), c_int64(k.stride(1)), c_int64(k.stride(0)),
        c_int64(v.stride(1)), c_int64(v.stride(0)), c_int64(o.stride(1)), c_int64(o.stride(0)),
        c_float(scale), c_int(1 if causal else 0), ptr(mask[0] if mask else None), ptr(mask[1] if mask else None),
        c_int(mask[0].shape[1] if mask else 0), ptr(_lib.status_buffer(q.device)), stream())
    check(rc, "pd_flash_attn_fwd")
    native._count()
    return o, lse


def bwd(do, q, k, v, o, lse, causal, scale, dq=None, dk=None, dv=None, mask=None):
    """Gradients of :func:`fwd`.  ``dq/dk/dv`` may be pre-allocated views (e.g. slices of one packed dqkv
    buffer); they only need dense 128-element heads."""
    q, k, v, o, do = (t if _view_ok(t) else t.contiguous() for t in (q, k, v, o, do))
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    dev = q.device
    dq = torch.empty((B, Sq, Hq, D), dtype=torch.bfloat16, device=dev) if dq is None else dq
    dk = torch.empty((B, Sk, Hkv, D), dtype=torch.bfloat16, device=dev) if dk is None else dk
    dv = torch.empty((B, Sk, Hkv, D), dtype=torch.bfloat16, device=dev) if dv is None else dv
    assert _view_ok(dq) and _view_ok(dk) and _view_ok(dv)
    dq_acc = torch.zeros((B, Sq, Hq, D), dtype=torch.float32, device=dev)
    delta = torch.empty((B, Hq, Sq), dtype=torch.float32, device=dev)
    rc = _lib.kernels().pd_flash_attn_bwd(
        ptr(do), ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), ptr(delta), ptr(dq_acc), ptr(None), ptr(dq), ptr(dk),
        ptr(dv), c_int(B), c_int(Sq), c_int(Sk), c_int(Hq), c_int(Hkv),
        c_int64(q.stride(1)), c_int64(q.stride(0)), c_int64(k.stride(1)), c_int64(k.stride(0)),
        c_int64(v.stride(1)), c_int64(v.stride(0)), c_int64(o.stride(1)), c_int64(o.stride(0)),
        c_int64(do.stride(1)), c_int64(do.stride(0)), c_int64(dq.stride(1)), c_int64(dq.stride(0)),
        c_int64(dk.stride(1)), c_int64(dk.stride(0)), c_int64(dv.stride(1)), c_int64(dv.stride(0)),
        c_float(scale), c_int(1 if causal else 0), ptr(mask[0] if mask else None), ptr(mask[1] if mask else None),
        c_int(mask[0].shape[1] if mask else 0), ptr(_lib.status_buffer(dev)), stream())
    check(rc, "pd_flash_attn_bwd")
    native._count(3)
    return dq, dk, dv


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, mask):
        o, lse = fwd(q, k, v, causal, scale, mask)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale, ctx.mask = causal, scale, mask
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = bwd(do, q, k, v, o, lse, ctx.causal, ctx.scale, mask=ctx.mask)
        return dq, dk, dv, None, None, None


def flash_attn_func(q, k, v, causal, scale, mask=None, return_lse=False):
    """``mask``: ``(bounds, tile_bounds)`` of :func:`normalize_flashmask` for column-sparse masking."""
    o, lse = _FlashAttnFn.apply(q, k, v, bool(causal), float(scale), mask)
    return (o, lse) if return_lse else o


class _RopeAttnPackedFn(torch.autograd.Function):
    """Rotary embedding + attention on a packed projection ``qkv[B*S, (Hq + 2 Hkv) * 128]``.

    Forward rotates the q and k heads inside the projection buffer itself (one launch: q and k heads are
    adjacent) and runs flash attention on views of that buffer; the un-rotated values are consumed — the
    producing linear layer never needs its own output again.  Backward lets the attention kernels write
    dq / dk / dv straight into one packed gradient buffer and un-rotates its q,k heads in place, so no slice,
    concat, zero-fill or gradient-accumulation kernel is launched for the projection."""

    @staticmethod
    def forward(ctx, qkv2d, cos, sin, B, S, hq, hkv, causal, scale):
        qkv = qkv2d.detach().view(B, S, hq + 2 * hkv, 128)
        rot = qkv[:, :, :hq + hkv]
        native.rope(rot, cos, sin, None, seq_len=S, half_style=True, out=rot)
        q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
        o, lse = fwd(q, k, v, causal, scale)
        ctx.save_for_backward(qkv, o, lse, cos, sin)
        ctx.meta = (B, S, hq, hkv, causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, cos, sin = ctx.saved_tensors
        B, S, hq, hkv, causal, scale = ctx.meta
        q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
        dqkv = torch.empty_like(qkv)
        bwd(do, q, k, v, o, lse, causal, scale, dq=dqkv[:, :, :hq], dk=dqkv[:, :, hq:hq + hkv],
            dv=dqkv[:, :, hq + hkv:])
        rot = dqkv[:, :, :hq + hkv]
        native.rope(rot, cos, sin, None, seq_len=S, half_style=True, backward=True, out=rot)
        return dqkv.view(B * S, -1), None, None, None, None, None, None, None, None


def rope_attention_packed(qkv2d, cos, sin, B, S, hq, hkv, causal, scale):
    """``qkv2d``: contiguous bf16 ``[B*S, (hq + 2*hkv) * 128]`` produced by the qkv projection (its q,k heads are
    overwritten with the rotated values).  Returns the attention output ``[B, S, hq, 128]``."""
    return _RopeAttnPackedFn.apply(qkv2d, cos, sin, int(B), int(S), int(hq), int(hkv), bool(causal), float(scale))
