"""Thin, allocation-explicit Python entry points for every native kernel.

Each function validates shapes/dtypes, allocates outputs with torch and calls the C ABI of
``libpd_kernels.so`` on the current stream.  Autograd wiring lives in ``paddle_b200.ops.functional``.
"""
from __future__ import annotations

import os

import ctypes

import torch

from . import _lib
from ._lib import c_float, c_int, c_int64, c_void_p, check, ptr, stream

BF16 = torch.bfloat16
F32 = torch.float32

LAUNCH_COUNT = 0  # number of native kernel launcher calls (bench.py reports it)


def _count(n: int = 1):
    global LAUNCH_COUNT
    LAUNCH_COUNT += n


def _req(cond: bool, msg: str):
    if not cond:
        raise ValueError(msg)


# --------------------------------------------------------------------------------------------- GEMM
EPI_BF16, EPI_F32, EPI_ACCUM_F32 = 0, 1, 2


# "1cta": 128 x 256 tile per SM (gemm_sm100.cu); "2cta": 256 x 256 tile per SM pair, tcgen05 cta_group::2
# (gemm2_sm100.cu).  PD_GEMM_IMPL selects; set_gemm_impl() switches at run time.
GEMM_IMPL = os.environ.get("PD_GEMM_IMPL", "2cta")     # measured 5-16 % faster on every Llama-2 7B shape and layout


def set_gemm_impl(name: str) -> str:
    global GEMM_IMPL
    _req(name in ("1cta", "2cta"), "gemm impl must be '1cta' or '2cta'")
    prev, GEMM_IMPL = GEMM_IMPL, name
    return prev


def gemm(a: torch.Tensor, b: torch.Tensor, trans_a: bool = False, trans_b: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype = BF16, accumulate: bool = False,
         max_ctas: int = 0) -> torch.Tensor:
    """``out (=|+=) op(a) @ op(b)`` on the tcgen05 tensor cores.

    ``a``/``b`` are 2-D bf16 with a unit inner stride.  ``op(a)`` is ``[M, K]`` (``a`` itself is
    ``[K, M]`` when ``trans_a``), ``op(b)`` is ``[K, N]`` (``b`` itself is ``[N, K]`` when ``trans_b``).
    ``accumulate=True`` requires an fp32 ``out`` and adds into it (TMA reduce-add epilogue).
    """
    _req(a.dtype == BF16 and b.dtype == BF16, "gemm: bf16 operands required")
    _req(a.dim() == 2 and b.dim() == 2, "gemm: 2-D operands required")
    _req(a.stride(1) == 1 and b.stride(1) == 1, "gemm: operands need a unit inner stride")
    M, K = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    Kb, N = (b.shape[1], b.shape[0]) if trans_b else (b.shape[0], b.shape[1])
    _req(K == Kb, f"gemm: inner dimensions differ ({K} vs {Kb})")
    if out is None:
        _req(not accumulate, "gemm: accumulate=True needs `out`")
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _req(out.shape[0] == M and out.shape[1] == N and out.stride(1) == 1, "gemm: bad `out`")
    if accumulate:
        _req(out.dtype == F32, "gemm: accumulate=True needs an fp32 `out`")
        epi = EPI_ACCUM_F32
    else:
        epi = EPI_BF16 if out.dtype == BF16 else EPI_F32
        _req(out.dtype in (BF16, F32), "gemm: out dtype must be bf16 or fp32")
    if GEMM_IMPL == "2cta":
        rc = _lib.kernels().pd_gemm_bf16_2cta(
            ptr(a), ptr(b), ptr(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)), c_int(b.stride(0)),
            c_int(out.stride(0)), c_int(1 if trans_a else 0), c_int(0 if trans_b else 1), c_int(epi),
            c_int(max_ctas), c_int(1), ptr(_lib.status_buffer(a.device)), stream())
        check(rc, "pd_gemm_bf16_2cta")
        _count()
        return out
    rc = _lib.kernels().pd_gemm_bf16(
        ptr(a), ptr(b), ptr(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)), c_int(b.stride(0)),
        c_int(out.stride(0)), c_int(1 if trans_a else 0), c_int(0 if trans_b else 1), c_int(epi),
        c_int(max_ctas), ptr(_lib.status_buffer(a.device)), stream())
    check(rc, "pd_gemm_bf16")
    _count()
    return out


# --------------------------------------------------------------------------------------------- norms
def rms_norm_fwd(x, w, eps, residual=None, want_residual_out=False):
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    _req(x2.dtype == BF16 and x2.is_contiguous(), "rms_norm: contiguous bf16 input required")
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    inv = torch.empty(rows, dtype=F32, device=x.device)
    res2 = residual.reshape(-1, H) if residual is not None else None
    res_out = torch.empty_like(x2) if (residual is not None and want_residual_out) else None
    rc = _lib.kernels().pd_rms_norm_fwd(ptr(x2), ptr(res2), ptr(w), c_int(1 if w.dtype == F32 else 0), ptr(y),
                                        ptr(res_out), ptr(inv), c_int64(rows), c_int(H), c_float(eps), stream())
    check(rc, "pd_rms_norm_fwd")
    _count()
    return y.view(x.shape), inv, (res_out.view(x.shape) if res_out is not None else None)


def rms_norm_bwd(dy, x, w, inv, dx_add=None, dw_out=None):
    """Returns (dx, dw_fp32).  ``dx_add`` is added into dx; ``dw_out`` (fp32) is accumulated into."""
    H = x.shape[-1]
    x2, dy2 = x.reshape(-1, H), dy.reshape(-1, H)
    _req(dy2.is_contiguous() and x2.is_contiguous(), "rms_norm_bwd: contiguous inputs required")
    rows = x2.shape[0]
    k = _lib.kernels()
    parts = k.pd_rms_norm_bwd_parts(c_int64(rows))
    partial = torch.empty((parts, H), dtype=F32, device=x.device)
    dx = torch.empty_like(x2)
    accumulate = dw_out is not None
    dw = dw_out if accumulate else torch.empty(H, dtype=F32, device=x.device)
    add2 = dx_add.reshape(-1, H) if dx_add is not None else None
    rc = k.pd_rms_norm_bwd(ptr(dy2), ptr(x2), ptr(w), c_int(1 if w.dtype == F32 else 0), ptr(inv), ptr(dx),
                           ptr(add2), ptr(partial), ptr(dw), c_int(1 if accumulate else 0), c_int64(rows),
                           c_int(H), stream())
    check(rc, "pd_rms_norm_bwd")
    _count(2)
    return dx.view(x.shape), dw


def layer_norm_fwd(x, w, b, eps):
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    _req(x2.dtype == BF16 and x2.is_contiguous(), "layer_norm: contiguous bf16 input required")
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    mean = torch.empty(rows, dtype=F32, device=x.device)
    rstd = torch.empty(rows, dtype=F32, device=x.device)
    rc = _lib.kernels().pd_layer_norm_fwd(ptr(x2), ptr(w), ptr(b), c_int(1 if w.dtype == F32 else 0), ptr(y),
                                          ptr(mean), ptr(rstd), c_int64(rows), c_int(H), c_float(eps), stream())
    check(rc, "pd_layer_norm_fwd")
    _count()
    return y.view(x.shape), mean, rstd


def layer_norm_bwd(dy, x, w, mean, rstd):
    H = x.shape[-1]
    x2, dy2 = x.reshape(-1, H), dy.reshape(-1, H).contiguous()
    rows = x2.shape[0]
    k = _lib.kernels()
    parts = k.pd_rms_norm_bwd_parts(c_int64(rows))
    pw = torch.empty((parts, H), dtype=F32, device=x.device)
    pb = torch.empty((parts, H), dtype=F32, device=x.device)
    dx = torch.empty_like(x2)
    dw = torch.empty(H, dtype=F32, device=x.device)
    db = torch.empty(H, dtype=F32, device=x.device)
    rc = k.pd_layer_norm_bwd(ptr(dy2), ptr(x2), ptr(w), c_int(1 if w.dtype == F32 else 0), ptr(mean), ptr(rstd),
                             ptr(dx), ptr(pw), ptr(pb), ptr(dw), ptr(db), c_int64(rows), c_int(H), stream())
    check(rc, "pd_layer_norm_bwd")
    _count(3)
    return dx.view(x.shape), dw, db


# --------------------------------------------------------------------------------------------- rope
def rope(x, cos, sin, position_ids=None, seq_len=None, half_style=True, backward=False, out=None):
    """x: [..., seq, heads, D] view whose last two dims are dense (token stride arbitrary)."""
    D = x.shape[-1]
    heads = x.shape[-2]
    _req(x.dtype == BF16 and x.stride(-1) == 1 and x.stride(-2) == D, "rope: need dense [heads, D] bf16 tail")
    tokens = x.numel() // (heads * D)
    tok_stride = x.stride(-3)
    # every leading dim must be expressible as token index * token stride
    xs = x.shape
    if x.dim() > 3:
        _req(all(x.stride(i) == x.stride(i + 1) * xs[i + 1] for i in range(x.dim() - 3)),
             "rope: leading dims must be collapsible")
    if out is None:
        out = torch.empty(xs, dtype=BF16, device=x.device)
    S = seq_len if seq_len is not None else xs[-3]
    _req(cos.dtype == F32 and sin.dtype == F32 and cos.shape[-1] == D, "rope: fp32 [pos, D] tables required")
    rc = _lib.kernels().pd_rope(ptr(x), ptr(out), ptr(cos), ptr(sin), ptr(position_ids), c_int64(tokens),
                                c_int(heads), c_int(D), c_int64(tok_stride), c_int64(out.stride(-3)), c_int(S),
                                c_int(1 if half_style else 0), c_int(1 if backward else 0), stream())
    check(rc, "pd_rope")
    _count()
    return out


# --------------------------------------------------------------------------------------------- swiglu
def swiglu_fwd(x, y=None):
    if y is None:
        F = x.shape[-1] // 2
        x2 = x.reshape(-1, 2 * F)
        _req(x2.is_contiguous(), "swiglu: contiguous input required")
        xa, ya, ld = x2, x2[:, F:], 2 * F
        out_shape = (*x.shape[:-1], F)
    else:
        F = x.shape[-1]
        xa, ya, ld = x.reshape(-1, F), y.reshape(-1, F), F
        _req(xa.is_contiguous() and ya.is_contiguous(), "swiglu: contiguous inputs required")
        out_shape = x.shape
    rows = xa.shape[0]
    out = torch.empty((rows, F), dtype=BF16, device=x.device)
    rc = _lib.kernels().pd_swiglu_fwd(ptr(xa), ptr(ya), ptr(out), c_int64(rows), c_int(F), c_int64(ld), stream())
    check(rc, "pd_swiglu_fwd")
    _count()
    return out.view(out_shape)


def swiglu_bwd(x, y, dout):
    if y is None:
        F = x.shape[-1] // 2
        x2 = x.reshape(-1, 2 * F)
        dx = torch.empty_like(x2)
        rows = x2.shape[0]
        d2 = dout.reshape(rows, F).contiguous()
        rc = _lib.kernels().pd_swiglu_bwd(ptr(x2), ptr(x2[:, F:]), ptr(d2), ptr(dx), ptr(dx[:, F:]), c_int64(rows),
                                          c_int(F), c_int64(2 * F), stream())
        check(rc, "pd_swiglu_bwd")
        _count()
        return dx.view(x.shape), None
    F = x.shape[-1]
    xa, ya = x.reshape(-1, F), y.reshape(-1, F)
    rows = xa.shape[0]
    d2 = dout.reshape(rows, F).contiguous()
    dx, dy = torch.empty_like(xa), torch.empty_like(ya)
    rc = _lib.kernels().pd_swiglu_bwd(ptr(xa), ptr(ya), ptr(d2), ptr(dx), ptr(dy), c_int64(rows), c_int(F),
                                      c_int64(F), stream())
    check(rc, "pd_swiglu_bwd")
    _count()
    return dx.view(x.shape), dy.view(y.shape)


# --------------------------------------------------------------------------------------------- CE
def ce_stats(logits2d, labels, vocab_start=0, ignore_index=-100, want_loss=True):
    """Row statistics (max, sum exp, target logit) and, for an unsharded vocab, the loss."""
    _req(logits2d.dim() == 2 and logits2d.is_contiguous(), "ce: contiguous [T, V] logits required")
    T, V = logits2d.shape
    dev = logits2d.device
    mx = torch.empty(T, dtype=F32, device=dev)
    sm = torch.empty(T, dtype=F32, device=dev)
    tg = torch.empty(T, dtype=F32, device=dev)
    loss = torch.empty(T, dtype=F32, device=dev) if want_loss else None
    labels = labels.reshape(-1).to(torch.int64)
    rc = _lib.kernels().pd_ce_stats(ptr(logits2d), c_int(1 if logits2d.dtype == F32 else 0), ptr(labels), ptr(mx),
                                    ptr(sm), ptr(tg), ptr(loss), c_int64(T), c_int(V), c_int64(vocab_start),
                                    c_int64(ignore_index), stream())
    check(rc, "pd_ce_stats")
    _count()
    return mx, sm, tg, loss


def ce_bwd(logits2d, labels, lse, dloss, vocab_start=0, ignore_index=-100, scale=1.0, inplace=False):
    T, V = logits2d.shape
    out = logits2d if inplace else torch.empty_like(logits2d)
    labels = labels.reshape(-1).to(torch.int64)
    dloss = dloss.to(F32).contiguous()
    rc = _lib.kernels().pd_ce_bwd(ptr(logits2d), c_int(1 if logits2d.dtype == F32 else 0), ptr(labels), ptr(lse),
                                  ptr(dloss), c_int(1 if dloss.numel() == 1 else 0), ptr(out), c_int64(T), c_int(V),
                                  c_int64(vocab_start), c_int64(ignore_index), c_float(scale), stream())
    check(rc, "pd_ce_bwd")
    _count()
    return out


# --------------------------------------------------------------------------------------------- embedding
def embedding_fwd(ids, table, vocab_start=0):
    H = table.shape[1]
    flat = ids.reshape(-1).to(torch.int64)
    out = torch.empty((flat.numel(), H), dtype=BF16, device=table.device)
    rc = _lib.kernels().pd_embedding_fwd(ptr(flat), ptr(table), ptr(out), c_int64(flat.numel()), c_int(H),
                                         c_int64(table.shape[0]), c_int64(vocab_start), stream())
    check(rc, "pd_embedding_fwd")
    _count()
    return out.view(*ids.shape, H)


def embedding_bwd(ids, dout, dtable_f32, vocab_start=0, padding_idx=-1):
    H = dtable_f32.shape[1]
    flat = ids.reshape(-1).to(torch.int64)
    d2 = dout.reshape(-1, H).contiguous()
    rc = _lib.kernels().pd_embedding_bwd(ptr(flat), ptr(d2), ptr(dtable_f32), c_int64(flat.numel()), c_int(H),
                                         c_int64(dtable_f32.shape[0]), c_int64(vocab_start), c_int64(padding_idx),
                                         stream())
    check(rc, "pd_embedding_bwd")
    _count()
    return dtable_f32


def accumulate_into_f32(src_bf16, acc_f32):
    rc = _lib.kernels().pd_accumulate_bf16_into_f32(ptr(src_bf16), ptr(acc_f32), c_int64(src_bf16.numel()), stream())
    check(rc, "pd_accumulate_bf16_into_f32")
    _count()
    return acc_f32


def add_bf16(a, b, out=None):
    out = torch.empty_like(a) if out is None else out
    rc = _lib.kernels().pd_add_bf16(ptr(a), ptr(b), ptr(out), c_int64(a.numel()), stream())
    check(rc, "pd_add_bf16")
    _count()
    return out


# --------------------------------------------------------------------------------------------- optimizer
class TensorTable:
    """Device-resident list of (param, grad, master, m, v) records consumed by the multi-tensor
    optimizer kernels.  Built once per parameter group; rebuilt only if a pointer changes."""

    def __init__(self, params, grads, masters=None, ms=None, vs=None):
        k = _lib.kernels()
        chunk = k.pd_opt_chunk_size()
        words = [len(params), 0]
        prefix = 0
        self.keepalive = (params, grads, masters, ms, vs)
        self._sig = []
        for i, p in enumerate(params):
            g = grads[i]
            n = p.numel()
            _req(p.is_contiguous() and g.is_contiguous() and g.numel() == n, "optimizer: contiguous tensors required")
            flags = (1 if p.dtype == BF16 else 0) | (2 if g.dtype == BF16 else 0)
            mp = masters[i] if masters is not None and masters[i] is not None else None
            if mp is not None:
                flags |= 4
            words += [n, prefix, p.data_ptr(), g.data_ptr(), mp.data_ptr() if mp is not None else 0,
                      ms[i].data_ptr() if ms is not None else 0, vs[i].data_ptr() if vs is not None else 0, flags]
            self._sig.append((p.data_ptr(), g.data_ptr()))
            prefix += (n + chunk - 1) // chunk
        words[1] = prefix
        self.total_chunks = prefix
        dev = params[0].device
        self.table = torch.tensor(words, dtype=torch.int64).to(dev)
        self.device = dev
        self._partial = None

    def matches(self, params, grads) -> bool:
        return len(params) == len(self._sig) and all(
            (p.data_ptr(), g.data_ptr()) == s for p, g, s in zip(params, grads, self._sig))

    def adamw(self, lr, beta1, beta2, eps, coeff, beta1_pow, beta2_pow, grad_scale=None, skip=None):
        rc = _lib.kernels().pd_adamw_multi(ptr(self.table), c_int64(self.total_chunks), c_float(lr), c_float(beta1),
                                           c_float(beta2), c_float(eps), c_float(coeff), c_float(beta1_pow),
                                           c_float(beta2_pow), ptr(grad_scale), ptr(skip), stream())
        check(rc, "pd_adamw_multi")
        _count()
        self._bump_versions()

    def momentum(self, lr, mu, wd, nesterov, use_momentum, grad_scale=None):
        rc = _lib.kernels().pd_momentum_multi(ptr(self.table), c_int64(self.total_chunks), c_float(lr), c_float(mu),
                                              c_float(wd), c_int(int(nesterov)), c_int(int(use_momentum)),
                                              ptr(grad_scale), stream())
        check(rc, "pd_momentum_multi")
        _count()
        self._bump_versions()

    def _bump_versions(self):
        """The kernels write the parameters through raw pointers; tell autograd (saved-tensor checks) and the caches
        keyed on a parameter's version (quantised weight copies) that their contents changed."""
        torch.autograd.graph.increment_version(self.keepalive[0])

    def sq_l2_norm(self, out=None, accumulate=False):
        k = _lib.kernels()
        if self._partial is None:
            self._partial = torch.empty(k.pd_l2norm_parts(c_int64(self.total_chunks)), dtype=F32, device=self.device)
        if out is None:
            out = torch.zeros(1, dtype=F32, device=self.device)
        rc = k.pd_sq_l2_norm_multi(ptr(self.table), c_int64(self.total_chunks), ptr(self._partial), ptr(out),
                                   c_int(1 if accumulate else 0), stream())
        check(rc, "pd_sq_l2_norm_multi")
        _count(2)
        return out

    def unscale_check(self, inv_scale, found_inf):
        rc = _lib.kernels().pd_unscale_check_multi(ptr(self.table), c_int64(self.total_chunks), ptr(inv_scale),
                                                   ptr(found_inf), stream())
        check(rc, "pd_unscale_check_multi")
        _count()


def adamw_flat(param_bf16, master, grad, m, v, lr, beta1, beta2, eps, coeff, beta1_pow, beta2_pow,
               grad_scale=None, skip=None):
    rc = _lib.kernels().pd_adamw_flat(ptr(param_bf16), ptr(master), ptr(grad), ptr(m), ptr(v), c_int64(master.numel()),
                                      c_float(lr), c_float(beta1), c_float(beta2), c_float(eps), c_float(coeff),
                                      c_float(beta1_pow), c_float(beta2_pow), ptr(grad_scale), ptr(skip), stream())
    check(rc, "pd_adamw_flat")
    _count()


# --------------------------------------------------------------------------------------------- decode / inference
ACT_CODES = {None: 0, "none": 0, "identity": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3, "silu": 4, "swish": 4}


def gemm_epilogue(a, b, bias=None, act=None, trans_a=False, trans_b=False, swiglu=False, out=None):
    """``act(op(a) @ op(b) + bias)`` in one kernel (bias bf16 ``[N]``; act in ``ACT_CODES``), or with ``swiglu=True``
    ``silu(gate) * up`` over the interleaved (gate, up) column pairs of the product, returning ``[M, N / 2]``."""
    _req(a.dtype == BF16 and b.dtype == BF16 and a.dim() == 2 and b.dim() == 2, "gemm_epilogue: 2-D bf16 operands required")
    _req(a.stride(1) == 1 and b.stride(1) == 1, "gemm_epilogue: operands need a unit inner stride")
    M, K = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    Kb, N = (b.shape[1], b.shape[0]) if trans_b else (b.shape[0], b.shape[1])
    _req(K == Kb, f"gemm_epilogue: inner dimensions differ ({K} vs {Kb})")
    _req(act in ACT_CODES, f"gemm_epilogue: unknown activation {act!r}")
    if bias is not None:
        _req(bias.dtype == BF16 and bias.numel() == N and bias.is_contiguous(), "gemm_epilogue: bias must be bf16 [N]")
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty((M, n_out), dtype=BF16, device=a.device)
    _req(out.dtype == BF16 and tuple(out.shape) == (M, n_out) and out.stride(1) == 1, "gemm_epilogue: bad `out`")
    rc = _lib.kernels().pd_gemm_bf16_2cta_epi(
        ptr(a), ptr(b), ptr(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)), c_int(b.stride(0)),
        c_int(out.stride(0)), c_int(1 if trans_a else 0), c_int(0 if trans_b else 1), ptr(bias), c_int(ACT_CODES[act]),
        c_int(1 if swiglu else 0), ptr(_lib.status_buffer(a.device)), stream())
    check(rc, "pd_gemm_bf16_2cta_epi")
    _count()
    return out


def dropout_add(x, y, p, upscale, seed, offset, out=None):
    """``dropout(x) [+ y]`` with keep decisions from the Philox stream at ``(seed, offset)``."""
    _req(x.is_contiguous() and x.dtype in (BF16, F32), "dropout_add: contiguous bf16 / fp32 input required")
    _req(y is None or (y.is_contiguous() and y.dtype == x.dtype and y.shape == x.shape), "dropout_add: bad `y`")
    out = torch.empty_like(x) if out is None else out
    rc = _lib.kernels().pd_dropout_add(ptr(x), ptr(y), ptr(out), c_int64(x.numel()), c_int(1 if x.dtype == F32 else 0),
                                       c_float(p), c_int(1 if upscale else 0), ctypes.c_ulonglong(int(seed) & (2 ** 64 - 1)),
                                       ctypes.c_ulonglong(int(offset)), stream())
    check(rc, "pd_dropout_add")
    _count()
    return out


def dropout_offset_step(n):
    k = _lib.kernels()
    k.pd_dropout_offset_step.restype = ctypes.c_longlong
    return int(k.pd_dropout_offset_step(c_int64(n)))


BIAS_ACT_CODES = {None: 0, "none": 0, "identity": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3, "silu": 4, "swish": 4,
                  "swiglu": 5, "geglu": 6}


def bias_act(x, bias, act):
    """``act(x + bias)`` over the last axis; ``swiglu`` / ``geglu`` halve it (gate half first)."""
    _req(x.dtype == BF16 and x.is_contiguous(), "bias_act: contiguous bf16 input required")
    code = BIAS_ACT_CODES[act]
    cols = x.shape[-1]
    F_ = cols // 2 if code >= 5 else cols
    rows = x.numel() // cols
    _req(bias is None or (bias.dtype == BF16 and bias.numel() == cols and bias.is_contiguous()), "bias_act: bad bias")
    out = torch.empty((*x.shape[:-1], F_), dtype=BF16, device=x.device)
    rc = _lib.kernels().pd_bias_act(ptr(x), ptr(bias), ptr(out), c_int64(rows), c_int(F_), c_int(code), stream())
    check(rc, "pd_bias_act")
    _count()
    return out


def sample_top_p_top_k(logits, top_p=None, top_k=0, temperature=1.0, seed=0, offset=0, input_is_prob=False,
                       draw_counter=None, out=None):
    """One token per row from ``softmax(logits / temperature)`` cut to the ``top_k`` most likely tokens and to the
    nucleus of mass ``top_p`` (fp32 ``[rows]`` or None).  Returns ``(ids int64 [rows], probs fp32 [rows])``."""
    _req(logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype in (BF16, F32), "sample: [rows, V] bf16 / fp32 required")
    rows, V = logits.shape
    ids = torch.empty(rows, dtype=torch.int64, device=logits.device) if out is None else out
    probs = torch.empty(rows, dtype=F32, device=logits.device)
    if top_p is not None:
        top_p = top_p.reshape(-1).to(F32).contiguous()
        _req(top_p.numel() == rows, "sample: one top_p per row required")
    rc = _lib.kernels().pd_sample_top_p_top_k(
        ptr(logits), c_int(1 if logits.dtype == F32 else 0), c_int64(rows), c_int64(logits.stride(0)), c_int(V), ptr(top_p),
        c_int(int(top_k)), c_float(float(temperature)), c_int(1 if input_is_prob else 0),
        ctypes.c_ulonglong(int(seed) & (2 ** 64 - 1)), ctypes.c_ulonglong(int(offset)), ptr(ids), ptr(probs), stream(),
        ptr(draw_counter))
    check(rc, "pd_sample_top_p_top_k")
    _count()
    return ids, probs


def gemm_splitk(a, b, acc_f32, splits=0, trans_b=False):
    """``acc_f32 += a @ op(b)`` with K cut into ``splits`` slices that run on different SMs (skinny decode GEMMs).
    ``splits=0`` picks a count that fills the GPU.  ``acc_f32`` must hold zeros (``splitk_finalize`` re-zeroes it)."""
    M, K = a.shape
    N = b.shape[0] if trans_b else b.shape[1]
    k = _lib.kernels()
    if splits <= 0:
        heuristic = k.pd_gemm_suggest_splits(c_int(M), c_int(N), c_int(K))
        from . import autotune
        if autotune._cfg["enable"]:
            def run(c):
                rc_ = k.pd_gemm_bf16_splitk(ptr(a), ptr(b), ptr(acc_f32), c_int(M), c_int(N), c_int(K),
                                            c_int(a.stride(0)), c_int(b.stride(0)), c_int(acc_f32.stride(0)), c_int(0),
                                            c_int(0 if trans_b else 1), c_int(c), ptr(_lib.status_buffer(a.device)), stream())
                check(rc_, "pd_gemm_bf16_splitk")
            cands = sorted({1, 2, 3, 4, 6, 8, heuristic} & set(range(1, max(2, K // 256) + 1)))
            tuned_before = autotune._stats["tuned"]
            splits = autotune.choose("gemm_splitk", (M, N, K, int(trans_b)), cands, run, heuristic)
            if autotune._stats["tuned"] != tuned_before:
                acc_f32.zero_()                    # the timing launches accumulated into it
        else:
            splits = heuristic
    rc = k.pd_gemm_bf16_splitk(ptr(a), ptr(b), ptr(acc_f32), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
                               c_int(b.stride(0)), c_int(acc_f32.stride(0)), c_int(0), c_int(0 if trans_b else 1),
                               c_int(splits), ptr(_lib.status_buffer(a.device)), stream())
    check(rc, "pd_gemm_bf16_splitk")
    _count()
    return acc_f32


def suggest_splits(M, N, K):
    return _lib.kernels().pd_gemm_suggest_splits(c_int(M), c_int(N), c_int(K))


def splitk_finalize(acc_f32, out=None, bias=None, residual=None):
    M, N = acc_f32.shape
    if out is None:
        out = torch.empty((M, N), dtype=BF16, device=acc_f32.device)
    rc = _lib.kernels().pd_splitk_finalize(ptr(acc_f32), ptr(bias), ptr(residual), ptr(out), c_int64(M), c_int(N),
                                           stream())
    check(rc, "pd_splitk_finalize")
    _count()
    return out


def decode_qkv_prep(qkv, bias, cos, sin, seq_lens, block_table, q_out, k_cache, v_cache, Hq, Hkv):
    B = qkv.shape[0]
    rc = _lib.kernels().pd_decode_qkv_prep(ptr(qkv), ptr(bias), ptr(cos), ptr(sin), ptr(seq_lens), ptr(block_table),
                                           ptr(q_out), ptr(k_cache), ptr(v_cache), c_int(B), c_int(Hq), c_int(Hkv),
                                           c_int(block_table.shape[1]), c_int64(qkv.stride(0)), c_int(cos.shape[0]),
                                           stream())
    check(rc, "pd_decode_qkv_prep")
    _count()
    return q_out


def write_kv_cache(k, v, block_table, k_cache, v_cache, start_pos=0):
    """k, v: [B, S, Hkv, 128] views (unit inner stride, head stride 128)."""
    B, S, Hkv, D = k.shape
    _req(D == 128 and k.stride(3) == 1 and k.stride(2) == 128 and v.stride() == k.stride(), "write_kv_cache: layout")
    rc = _lib.kernels().pd_write_kv_cache(ptr(k), ptr(v), ptr(block_table), ptr(k_cache), ptr(v_cache), c_int(B),
                                          c_int(S), c_int(Hkv), c_int(block_table.shape[1]), c_int64(k.stride(1)),
                                          c_int64(k.stride(0)), c_int(start_pos), stream())
    check(rc, "pd_write_kv_cache")
    _count()


def decode_attn_splits(B, Hkv, max_pages):
    return _lib.kernels().pd_decode_attn_splits(c_int(B), c_int(Hkv), c_int(max_pages))


def paged_decode_attn(q, k_cache, v_cache, block_table, seq_lens, scale, out=None, nsplit=1, len_offset=0,
                      workspace=None):
    """q [B, Hq, 128] bf16; caches [num_blocks, Hkv, 64, 128]; block_table [B, max_blocks] int32; seq_lens [B] int32."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    _req(D == 128 and q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous(), "paged attn: layout")
    if out is None:
        out = torch.empty_like(q)
    pa = pm = None
    if nsplit > 1:
        if workspace is None:
            workspace = (torch.empty((B, Hq, nsplit, 128), dtype=F32, device=q.device),
                         torch.empty((B, Hq, nsplit, 2), dtype=F32, device=q.device))
        pa, pm = workspace
    rc = _lib.kernels().pd_paged_decode_attn(ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_table), ptr(seq_lens),
                                             ptr(out), ptr(pa), ptr(pm), c_int(B), c_int(Hq), c_int(Hkv),
                                             c_int(block_table.shape[1]), c_int(nsplit), c_int(len_offset),
                                             c_float(scale), ptr(_lib.status_buffer(q.device)), stream())
    check(rc, "pd_paged_decode_attn")
    _count(2 if nsplit > 1 else 1)
    return out


# --------------------------------------------------------------------------------------------- MoE / fp8
def moe_topk_softmax(logits, k, normalize=True, counts=None):
    """logits [T, E] fp32 -> (weights [T, k] fp32, indices [T, k] int32); ``counts`` [E] int32 is incremented."""
    T, E = logits.shape
    lg = logits.float().contiguous()
    w = torch.empty((T, k), dtype=F32, device=lg.device)
    idx = torch.empty((T, k), dtype=torch.int32, device=lg.device)
    rc = _lib.kernels().pd_moe_topk_softmax(ptr(lg), c_int(T), c_int(E), c_int(k), c_int(1 if normalize else 0), ptr(w),
                                            ptr(idx), ptr(counts), stream())
    check(rc, "pd_moe_topk_softmax")
    _count()
    return w, idx


def fp8_quant_1x128(x):
    """bf16 [T, H] -> (e4m3 [T, H], fp32 scales [T, H/128]); dequantised value = q * scale."""
    T, H = x.shape
    _req(x.dtype == BF16 and x.is_contiguous() and H % 128 == 0, "fp8_quant_1x128: contiguous bf16 with H % 128 == 0")
    q = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((T, H // 128), dtype=F32, device=x.device)
    rc = _lib.kernels().pd_fp8_quant_1x128(ptr(x), ptr(q), ptr(s), c_int64(T), c_int(H), stream())
    check(rc, "pd_fp8_quant_1x128")
    _count()
    return q, s


def fp8_quant_weight(w):
    """bf16 W [K, N] (or [E, K, N]) -> (e4m3 W^T [.., N, K], fp32 scales [.., K/128, N/128]) with 128 x 128 blocks."""
    ws = w if w.dim() == 3 else w[None]
    E, K, N = ws.shape
    _req(ws.dtype == BF16 and ws.is_contiguous() and K % 128 == 0 and N % 128 == 0, "fp8_quant_weight: K, N % 128 == 0")
    q = torch.empty((E, N, K), dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty((E, K // 128, N // 128), dtype=F32, device=w.device)
    for e in range(E):
        rc = _lib.kernels().pd_fp8_quant_128x128_t(ptr(ws[e]), ptr(q[e]), ptr(s[e]), c_int(K), c_int(N), stream())
        check(rc, "pd_fp8_quant_128x128_t")
    _count(E)
    return (q, s) if w.dim() == 3 else (q[0], s[0])


def grouped_gemm_fp8(a_q, a_scale, b_q, b_scale, offsets, out=None):
    """Tokens sorted by expert: rows ``offsets[e]:offsets[e+1]`` of ``a_q`` [M, K] multiply expert ``e`` of
    ``b_q`` [E, N, K]; returns bf16 [M, N].  ``offsets`` is an int32 device tensor of length E + 1."""
    M, K = a_q.shape
    E, N, _ = b_q.shape
    if out is None:
        out = torch.empty((M, N), dtype=BF16, device=a_q.device)
    max_tiles = ((M + 127) // 128 + E) * (N // 128)
    rc = _lib.kernels().pd_grouped_gemm_fp8(ptr(a_q), ptr(a_scale), ptr(b_q), ptr(b_scale), ptr(offsets), ptr(out),
                                            c_int(M), c_int(N), c_int(K), c_int(E), c_int(out.stride(0)), c_int(max_tiles),
                                            ptr(_lib.status_buffer(a_q.device)), stream())
    check(rc, "pd_grouped_gemm_fp8")
    _count()
    return out
