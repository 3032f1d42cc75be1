"""Kernel micro-benchmarks: ``python -m paddle_b200.ops.kernel_bench --op gemm|attention|norm|adamw|all``.

Every kernel is timed with CUDA events on the launching stream after three warm-up launches; between timed
launches a buffer larger than L2 is overwritten so operands come from HBM.  Each line reports the achieved
FLOP/s or bytes/s and its fraction of the measured peaks (a STREAM-style copy and a cuBLAS bf16 GEMM measured
on the same GPU model; ``--peaks`` names the JSON that holds them), next to the library kernel for the same
shape (cuBLAS, cuDNN/flash SDPA, torch foreach) as the baseline.

``--small`` shrinks the shapes (inputs still larger than L2 where bandwidth matters) so that one launch can be
captured by a profiler in seconds; ``--iters`` and ``--only NAME`` restrict what runs.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks(path):
    hbm, tf = 6650.0, 1590.0
    try:
        with open(path) as f:
            d = json.load(f)
        hbm = float(d.get("hbm_gbs", hbm))
        tf = float(d.get("bf16_tflops", tf))
    except (OSError, ValueError):
        pass
    return hbm, tf


class _Timer:
    def __init__(self, flush=True):
        self.flush_buf = torch.empty(160 << 20, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn, iters=10, warmup=3):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(iters):
            if self.flush_buf is not None:
                self.flush_buf.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        return total / iters


def bench_gemm(args, timer, hbm, tf):
    from . import native
    shapes = [(4096, 4096, 4096, False, False, "fwd_qkvo"), (4096, 22016, 4096, False, False, "fwd_gateup"),
              (4096, 4096, 11008, False, False, "fwd_down"), (4096, 4096, 4096, False, True, "dgrad"),
              (4096, 11008, 4096, True, False, "wgrad"), (4096, 32000, 4096, False, False, "lm_head"),
              (8192, 8192, 8192, False, True, "sq8k_nt")]
    if args.small:
        shapes = [(2048, 4096, 4096, False, False, "small_nn"), (2048, 4096, 4096, False, True, "small_nt")]
    out = []
    for M, N, K, ta, tb, name in shapes:
        if args.only and name != args.only:
            continue
        a = torch.randn((K, M) if ta else (M, K), device="cuda").to(torch.bfloat16)
        b = torch.randn((N, K) if tb else (K, N), device="cuda").to(torch.bfloat16)
        t = timer(lambda: native.gemm(a, b, ta, tb), args.iters)
        # the other tile scheme for comparison (default: 256 x 256 per SM pair, cta_group::2)
        other = "1cta" if native.GEMM_IMPL == "2cta" else "2cta"
        prev = native.set_gemm_impl(other)
        t_other = timer(lambda: native.gemm(a, b, ta, tb), args.iters)
        native.set_gemm_impl(prev)
        A, B = (a.t() if ta else a), (b.t() if tb else b)
        t2 = timer(lambda: torch.matmul(A, B), args.iters) if not args.no_baseline else float("nan")
        fl = 2.0 * M * N * K
        out.append(dict(op="gemm", name=name, impl=prev, M=M, N=N, K=K, ms=t, tflops=fl / t / 1e9,
                        frac_of_measured=fl / t / 1e9 / tf, **{f"{other}_ms": t_other, f"{other}_tflops": fl / t_other / 1e9},
                        lib_ms=t2, lib_tflops=fl / t2 / 1e9))
        print(json.dumps(out[-1]), flush=True)
    return out


def bench_attention(args, timer, hbm, tf):
    from . import attention
    B, S, H, D = (1, 2048, 8, 128) if args.small else (1, 4096, 32, 128)
    qkv = torch.randn(B, S, 3 * H, D, device="cuda").to(torch.bfloat16)
    q, k, v = qkv[:, :, :H], qkv[:, :, H:2 * H], qkv[:, :, 2 * H:]
    scale = D ** -0.5
    out = []
    for causal in (True, False):
        name = "causal" if causal else "full"
        if args.only and name != args.only:
            continue
        fl = 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)
        t = timer(lambda: attention.fwd(q, k, v, causal, scale), args.iters)
        o, lse = attention.fwd(q, k, v, causal, scale)
        do = torch.randn_like(o)
        tb = timer(lambda: attention.bwd(do, q, k, v, o, lse, causal, scale), args.iters)
        rec = dict(op="attention", name=name, B=B, S=S, H=H, D=D, fwd_ms=t, fwd_tflops=fl / t / 1e9,
                   fwd_frac_of_measured=fl / t / 1e9 / tf, bwd_ms=tb, bwd_tflops=2.5 * fl / tb / 1e9,
                   bwd_frac_of_measured=2.5 * fl / tb / 1e9 / tf)
        if not args.no_baseline:
            qh, kh, vh = (x.transpose(1, 2).detach().requires_grad_() for x in (q, k, v))
            t2 = timer(lambda: torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=scale),
                       args.iters)
            oo = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=scale)
            go = torch.randn_like(oo)
            t3 = timer(lambda: torch.autograd.grad(oo, (qh, kh, vh), go, retain_graph=True), args.iters)
            rec.update(lib_fwd_ms=t2, lib_fwd_tflops=fl / t2 / 1e9, lib_bwd_ms=t3, lib_bwd_tflops=2.5 * fl / t3 / 1e9)
        out.append(rec)
        print(json.dumps(rec), flush=True)
    return out


def bench_norm(args, timer, hbm, tf):
    from . import native
    T, H = (16384, 4096) if args.small else (65536, 4096)      # 128 MiB / 512 MiB of bf16 activations
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    out = []
    t = timer(lambda: native.rms_norm_fwd(x, w, 1e-6), args.iters)
    by = 2.0 * x.numel() * 2
    rec = dict(op="rms_norm_fwd", T=T, H=H, ms=t, gbs=by / t / 1e6, frac_of_measured=by / t / 1e6 / hbm)
    if not args.no_baseline:
        t2 = timer(lambda: torch.nn.functional.rms_norm(x, (H,), w, 1e-6), args.iters)
        rec.update(lib_ms=t2, lib_gbs=by / t2 / 1e6)
    out.append(rec)
    print(json.dumps(rec), flush=True)
    gu = torch.randn(T, 2 * H, device="cuda").to(torch.bfloat16)
    t = timer(lambda: native.swiglu_fwd(gu), args.iters)
    by = 3.0 * T * H * 2
    rec = dict(op="swiglu_fwd", T=T, H=H, ms=t, gbs=by / t / 1e6, frac_of_measured=by / t / 1e6 / hbm)
    out.append(rec)
    print(json.dumps(rec), flush=True)
    return out


def bench_adamw(args, timer, hbm, tf):
    from . import native
    n = (64 << 20) if args.small else (512 << 20)     # elements; bf16 param + fp32 master/m/v/grad = 18 B each
    p = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    master, m, v = (torch.zeros(n, device="cuda", dtype=torch.float32) for _ in range(3))
    g = torch.full((n,), 1e-3, device="cuda", dtype=torch.float32)
    step = [0]

    def run():
        step[0] += 1
        native.adamw_flat(p, master, g, m, v, 1e-4, 0.9, 0.95, 1e-8, 0.01, 0.9 ** step[0], 0.95 ** step[0])
    t = timer(run, args.iters)
    by = n * (4 + 3 * 8 + 2.0)      # read grad; read+write master, m, v; write bf16 param
    rec = dict(op="adamw_flat", n=n, ms=t, gbs=by / t / 1e6, frac_of_measured=by / t / 1e6 / hbm)
    print(json.dumps(rec), flush=True)
    out = [rec]
    # the multi-tensor form the optimizers use: a list of Llama-sized matrices behind one device table
    shapes = [(4096, 12288), (4096, 4096), (4096, 22016), (11008, 4096)] * (1 if args.small else 8)
    ps = [torch.zeros(s, device="cuda", dtype=torch.bfloat16) for s in shapes]
    gs = [torch.full(s, 1e-3, device="cuda", dtype=torch.float32) for s in shapes]
    ma, ms, vs = ([torch.zeros(s, device="cuda", dtype=torch.float32) for s in shapes] for _ in range(3))
    tab = native.TensorTable(ps, gs, ma, ms, vs)
    n = sum(p.numel() for p in ps)

    def run_multi():
        step[0] += 1
        tab.adamw(1e-4, 0.9, 0.95, 1e-8, 0.01, 0.9 ** step[0], 0.95 ** step[0])
    t = timer(run_multi, args.iters)
    by = n * (4 + 3 * 8 + 2.0)
    rec = dict(op="adamw_multi", n=n, tensors=len(ps), ms=t, gbs=by / t / 1e6, frac_of_measured=by / t / 1e6 / hbm)
    print(json.dumps(rec), flush=True)
    out.append(rec)
    t = timer(lambda: tab.sq_l2_norm(), args.iters)
    rec = dict(op="sq_l2_norm_multi", n=n, ms=t, gbs=n * 4.0 / t / 1e6, frac_of_measured=n * 4.0 / t / 1e6 / hbm)
    print(json.dumps(rec), flush=True)
    out.append(rec)
    return out


def bench_decode(args, timer, hbm, tf):
    """Paged decode attention (bandwidth-bound: every cached K/V byte is read once) and the skinny split-K GEMM."""
    import math

    from . import native
    B, H, ctx = (16, 8, 1024) if args.small else (64, 40, 1280)
    pages = (ctx + 63) // 64
    nblocks = B * pages
    kc = torch.randn(nblocks, H, 64, 128, device="cuda").to(torch.bfloat16)
    vc = torch.randn(nblocks, H, 64, 128, device="cuda").to(torch.bfloat16)
    q = torch.randn(B, H, 128, device="cuda").to(torch.bfloat16)
    table = torch.randperm(nblocks, device="cuda").int().reshape(B, pages)
    lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    nsplit = native.decode_attn_splits(B, H, pages)
    out = []
    t = timer(lambda: native.paged_decode_attn(q, kc, vc, table, lens, 1 / math.sqrt(128), nsplit=nsplit), args.iters)
    by = 2.0 * B * ctx * H * 128 * 2
    rec = dict(op="paged_decode_attn", B=B, heads=H, ctx=ctx, nsplit=nsplit, ms=t, gbs=by / t / 1e6,
               frac_of_measured=by / t / 1e6 / hbm)
    print(json.dumps(rec), flush=True)
    out.append(rec)
    M = 64
    for name, K_, N in (("out_proj", 5120, 5120), ("ffn2", 13824, 5120), ("qkv", 5120, 15360), ("ffn1", 5120, 27648)):
        if args.small and name != "out_proj":
            continue
        x = torch.randn(M, K_, device="cuda").to(torch.bfloat16)
        w = (torch.randn(K_, N, device="cuda") * 0.02).to(torch.bfloat16)
        s = native.suggest_splits(M, N, K_)
        acc = torch.zeros(M, N, device="cuda", dtype=torch.float32)

        def run():
            if s > 1:
                native.gemm_splitk(x, w, acc, s)
                native.splitk_finalize(acc)
            else:
                native.gemm(x, w)
        t = timer(run, args.iters)
        by = 2.0 * K_ * N
        rec = dict(op="skinny_gemm", name=name, M=M, N=N, K=K_, splits=s, ms=t, gbs=by / t / 1e6,
                   frac_of_measured=by / t / 1e6 / hbm)
        if not args.no_baseline:
            t2 = timer(lambda: torch.matmul(x, w), args.iters)
            rec.update(lib_ms=t2, lib_gbs=by / t2 / 1e6)
        print(json.dumps(rec), flush=True)
        out.append(rec)
    return out


def bench_moe(args, timer, hbm, tf):
    """Grouped block-scaled fp8 expert GEMM (all experts in one launch) against the per-expert bf16 GEMM loop."""
    from . import native
    E, M, K_, N = (4, 8192, 4096, 8192) if args.small else (8, 16384, 4096, 28672)
    per = M // E
    x = torch.randn(M, K_, device="cuda").to(torch.bfloat16)
    w = (torch.randn(E, K_, N, device="cuda") * 0.02).to(torch.bfloat16)
    offs = torch.arange(0, M + 1, per, dtype=torch.int32, device="cuda")
    xq, xs = native.fp8_quant_1x128(x)
    wq, ws = native.fp8_quant_weight(w)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    fl = 2.0 * M * K_ * N
    t = timer(lambda: native.grouped_gemm_fp8(xq, xs, wq, ws, offs, out=out), args.iters)
    tq = timer(lambda: native.fp8_quant_1x128(x), args.iters)
    rec = dict(op="grouped_gemm_fp8", E=E, M=M, K=K_, N=N, ms=t, tflops=fl / t / 1e9, frac_of_measured_bf16_peak=fl / t / 1e9 / tf,
               act_quant_ms=tq)
    if not args.no_baseline:
        def loop():
            for e in range(E):
                native.gemm(x[e * per:(e + 1) * per], w[e], out=out[e * per:(e + 1) * per])
        t2 = timer(loop, args.iters)
        rec.update(bf16_loop_ms=t2, bf16_loop_tflops=fl / t2 / 1e9)
    print(json.dumps(rec), flush=True)
    return [rec]


def bench_fused_gemm(args, timer, hbm, tf):
    """Tensor-core side of the fused all-gather -> GEMM kernel on one GPU: the gathered operand is complete in the
    staging buffer (no pushes, no flag waits), so the number isolates what the fused kernel's tile loop costs
    against the plain GEMM on the same shape."""
    import ctypes

    from . import _lib, native
    from ._lib import c_int, ptr, stream
    T, H, N = (2048, 4096, 4096) if args.small else (4096, 4096, 6144)
    k = _lib.kernels()
    xfull = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    x = xfull[: T // 2].contiguous()
    w = (torch.randn(H, N, device="cuda") * 0.05).to(torch.bfloat16)
    y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(1024, dtype=torch.int32, device="cuda")
    ack = torch.zeros(16, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    U = ctypes.c_ulonglong * 8
    ps, pf, pa = U(*([xfull.data_ptr()] * 8)), U(*([flags.data_ptr()] * 8)), U(*([ack.data_ptr()] * 8))

    def ag():
        rc = k.pd_ag_gemm(ptr(xfull), ptr(w), ptr(y), c_int(T), c_int(N), c_int(H), c_int(H), c_int(N), c_int(N), c_int(0),
                          c_int(1), c_int(0), c_int(0), ptr(x), c_int(T // 2), c_int(128), c_int(H), c_int(0), c_int(2),
                          c_int(0), c_int(0), c_int(0), c_int(1), c_int(0), ps, pf, pa, ptr(done), c_int(0), None, c_int(2000),
                          c_int(0), c_int(1), ctypes.c_ulonglong(0), ptr(_lib.status_buffer()), stream())
        _lib.check(rc, "pd_ag_gemm")
    fl = 2.0 * T * N * H
    t = timer(ag, args.iters)
    t2 = timer(lambda: native.gemm(xfull, w), args.iters)
    rec = dict(op="ag_gemm_tile_loop", M=T, N=N, K=H, ms=t, tflops=fl / t / 1e9, frac_of_measured=fl / t / 1e9 / tf,
               plain_gemm_ms=t2, plain_gemm_tflops=fl / t2 / 1e9)
    print(json.dumps(rec), flush=True)
    out = [rec]
    # GEMM -> reduce-scatter kernel as a group of ONE rank: partial tiles go through the receive buffer and the
    # reduction pass on the same GPU, so the number shows what the kernel's own structure costs without any link
    M2, N2, K2 = (2048, 4096, 2048) if args.small else (4096, 4096, 2048)
    a = torch.randn(M2, K2, device="cuda").to(torch.bfloat16)
    b = (torch.randn(K2, N2, device="cuda") * 0.05).to(torch.bfloat16)
    o = torch.empty(M2, N2, device="cuda", dtype=torch.bfloat16)
    recv = torch.zeros(M2 * N2, device="cuda", dtype=torch.bfloat16)
    cnt = torch.zeros(((M2 + 127) // 128) * ((N2 + 255) // 256) + 8, dtype=torch.int32, device="cuda")
    ack2 = torch.zeros(16, dtype=torch.int32, device="cuda")
    done2 = torch.zeros(1, dtype=torch.int32, device="cuda")
    pr, pc, pa2 = U(*([recv.data_ptr()] * 8)), U(*([cnt.data_ptr()] * 8)), U(*([ack2.data_ptr()] * 8))
    ep = [0]

    def rs():
        ep[0] += 1
        rc = k.pd_gemm_rs(ptr(a), ptr(b), ptr(o), c_int(M2), c_int(N2), c_int(K2), c_int(K2), c_int(N2), c_int(0), c_int(1),
                          c_int(M2), c_int(0), c_int(1), c_int(ep[0]), pr, pc, pa2, ptr(done2), None, c_int(2000),
                          ptr(_lib.status_buffer()), stream())
        _lib.check(rc, "pd_gemm_rs")
    fl = 2.0 * M2 * N2 * K2
    t = timer(rs, args.iters)
    t2 = timer(lambda: native.gemm(a, b), args.iters)
    _lib.check_status()
    ok = bool(torch.equal(o, native.gemm(a, b)))
    rec = dict(op="gemm_rs_single_rank", M=M2, N=N2, K=K2, ms=t, tflops=fl / t / 1e9, frac_of_measured=fl / t / 1e9 / tf,
               plain_gemm_ms=t2, plain_gemm_tflops=fl / t2 / 1e9, matches_plain_gemm=ok)
    print(json.dumps(rec), flush=True)
    out.append(rec)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["gemm", "attention", "norm", "adamw", "decode", "fused_gemm", "moe", "all"])
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-baseline", action="store_true")
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--peaks", default=os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__)))), "MEASURED_PEAKS.json"))
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    from . import _lib
    hbm, tf = _peaks(args.peaks)
    timer = _Timer(flush=not args.no_flush)
    res = []
    for name, fn in (("gemm", bench_gemm), ("attention", bench_attention), ("norm", bench_norm), ("adamw", bench_adamw),
                     ("decode", bench_decode), ("fused_gemm", bench_fused_gemm), ("moe", bench_moe)):
        if args.op in (name, "all"):
            res += fn(args, timer, hbm, tf)
    _lib.check_status()
    if args.out:
        with open(args.out, "w") as f:
            json.dump({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf}, "results": res}, f, indent=1)
    return res


if __name__ == "__main__":
    main()
