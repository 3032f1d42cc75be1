"""Per-kernel timing of the fused all-gather->GEMM / GEMM->reduce-scatter kernels against the unfused sequence
(cuBLAS GEMM + NCCL collective on the same tensors), one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29500 \
        -m paddle_b200.parallel.bench_fused_comm [--hidden 4096] [--ffn 11008] [--tokens 4096] [--iters 30] [--sweep]

Shapes are the Llama-2 7B tensor-parallel linears at degree N (qkv / gate_up: column parallel, all-gather in front;
o_proj / down: row parallel, reduce-scatter behind).  Times are CUDA events on the launching stream after warm-up,
max over ranks.  ``--extra`` adds the decode GEMM->all-reduce, the gradient-bucket reduce-scatter (+AdamW) and the stage-3 linear against
their unfused sequences.  ``--sweep`` also times every push form (bulk ring / vector stores / multicast) with several push-CTA
counts and the NVLS reduce-scatter with several reducer counts.  Rank 0 prints one JSON object per line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--extra", action="store_true",
                    help="also time the decode GEMM->all-reduce, the bucket reduce-scatter (+AdamW) and the stage-3 linear")
    ap.add_argument("--trace", action="store_true",
                    help="print the per-CTA phase timestamps of the push reduce-scatter GEMM (GEMM tiles done, arrivals "
                         "published, first reduce unit, reduction done; microseconds from kernel start)")
    args = ap.parse_args()

    import torch.distributed as tdist

    import paddle_b200 as paddle
    from paddle_b200.distributed import fleet
    from paddle_b200.distributed.fleet.utils import sequence_parallel_utils as spu
    from paddle_b200.ops import _lib, native
    from paddle_b200.parallel import fused_linear_impl as FL

    n = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    paddle.set_device(f"gpu:{local}")
    st = fleet.DistributedStrategy()
    st.hybrid_configs = {"dp_degree": 1, "mp_degree": n, "pp_degree": 1, "sharding_degree": 1}
    fleet.init(is_collective=True, strategy=st)
    rank = tdist.get_rank()
    g = fleet.get_hybrid_communicate_group().get_model_parallel_group()
    T, H = args.tokens, args.hidden
    rows = T // n
    torch.manual_seed(7 + rank)

    def timed(fn):
        for _ in range(5):
            fn()
        tdist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / args.iters], device="cuda")
        tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
        _lib.check_status()
        return float(t) * 1e3      # us

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))

    def emit(rec):
        if rank == 0:
            print(json.dumps(rec), flush=True)

    mc = FL._AGSlot(g, 128, 64).mc_stage != 0
    emit({"ranks": n, "tokens": T, "hidden": H, "multicast": mc})
    col_shapes = {"qkv": 3 * H // n, "gate_up": (2 * args.ffn // n) // 8 * 8}
    row_shapes = {"o_proj": H // n, "down": (args.ffn // n) // 8 * 8}

    def ag_pair(mode):
        os.environ["PD_AG_PUSH_MODE"] = str(mode)
        pair = [FL._AGSlot(g, rows, H), FL._AGSlot(g, rows, H)]
        os.environ.pop("PD_AG_PUSH_MODE")
        return pair

    def rs_pair(use_mc, n_red, N):
        os.environ["PD_RS_MODE"] = "1" if use_mc else "0"
        os.environ["PD_RS_RED_CTAS"] = str(n_red)
        pair = [FL._RSSlot(g, rows, N), FL._RSSlot(g, rows, N)]
        os.environ.pop("PD_RS_MODE"), os.environ.pop("PD_RS_RED_CTAS")
        return pair

    modes = [0, 1] + ([2] if mc else [])
    for name, N in col_shapes.items():
        x = (torch.randn(rows, H, device="cuda") * 0.5).to(torch.bfloat16)
        w = (torch.randn(H, N, device="cuda") * 0.05).to(torch.bfloat16)
        y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        xfull = spu.all_gather(x, g)
        ref = torch.matmul(xfull, w)
        rec = {"op": f"ag_gemm_{name}", "shape": [T, H, N],
               "cublas_us": timed(lambda: torch.matmul(xfull, w)),
               "plain_gemm_us": timed(lambda: native.gemm(xfull, w)),
               "nccl_ag_us": timed(lambda: spu.all_gather(x, g)),
               "unfused_us": timed(lambda: torch.matmul(spu.all_gather(x, g), w)),
               "compute_bound_us": 2.0 * T * H * N / 1644e12 * 1e6,
               "link_bound_us": (n - 1) * rows * H * 2 / 770e9 * 1e6}
        configs = [(m, None) for m in modes]
        if args.sweep:
            configs += [(m, c) for m in modes for c in (4, 8, 16, 32, 48)]
        for mode, ctas in configs:
            pair = ag_pair(mode)
            state = {"i": 0}
            if ctas is not None:
                os.environ["PD_AG_COMM_CTAS"] = str(ctas)
                FL.N_COMM = ctas

            def run():
                s = pair[state["i"] & 1]
                state["i"] += 1
                FL.ag_gemm(s, g, x, s.stage, w, y, T, N, H, 0, 1, 0, 0)
            y.zero_()
            run()
            torch.cuda.synchronize()
            err = rel(y, ref)
            t = timed(run)
            os.environ.pop("PD_AG_COMM_CTAS", None)
            key = f"fused_mode{mode}" + (f"_ctas{ctas}" if ctas is not None else "")
            rec[key + "_us"] = t
            rec[key + "_err"] = err
            if args.trace and ctas is None:
                import ctypes

                import numpy as np
                k = _lib.kernels()
                k.pd_ag_gemm_trace(1)
                for _ in range(3):
                    run()
                torch.cuda.synchronize()
                tdist.barrier()
                buf = (ctypes.c_ulonglong * 2048)()
                k.pd_ag_gemm_trace_read(buf)
                k.pd_ag_gemm_trace(0)
                tt = np.array(list(buf), dtype=np.float64).reshape(256, 8)
                gemm = tt[tt[:, 3] > 0]
                comm = tt[tt[:, 4] > 0]
                if gemm.size:
                    t0 = gemm[:, 0].min()
                    med = lambda v: [round(float(v.min()), 1), round(float(np.median(v)), 1), round(float(v.max()), 1)]   # noqa: E731
                    rec[key + "_trace"] = {"gemm_ctas": int(gemm.shape[0]), "comm_ctas": int(comm.shape[0]),
                                           "loads_issued_us": med((gemm[:, 1] - t0) / 1e3),
                                           "flag_wait_us": med(gemm[:, 2] / 1e3),
                                           "epilogue_done_us": med((gemm[:, 3] - t0) / 1e3),
                                           "push_done_us": med((comm[:, 4] - t0) / 1e3) if comm.size else None}
                for r_ in range(8 * 256):
                    buf[r_] = 0
            del pair
        emit(rec)
        # weight gradient of the same layer: dW += gather(x)^T dY with the gathered x already staged (no push), once
        # through the flag-driven all-gather GEMM kernel and once as a plain GEMM over the staging buffer
        slot = FL._AGSlot(g, rows, H)
        FL.ag_gemm(slot, g, x, slot.stage, w, y, T, N, H, 0, 1, 0, 0, push=True, ack=False)
        slot.stage[rank * rows:(rank + 1) * rows].copy_(x)
        torch.cuda.synchronize()
        tdist.barrier()
        dy = (torch.randn(T, N, device="cuda") * 0.05).to(torch.bfloat16)
        mg = torch.zeros(H, N, device="cuda", dtype=torch.float32)
        ref_dw = xfull.float().t() @ dy.float()
        FL.ag_gemm(slot, g, x, slot.stage, dy, mg, H, N, T, 1, 1, 2, 1, False, False, False)
        err_ag = rel(mg, ref_dw)
        mg.zero_()
        native.gemm(slot.stage, dy, trans_a=True, out=mg, accumulate=True)
        err_plain = rel(mg, ref_dw)
        wrec = {"op": f"wgrad_{name}", "shape": [H, N, T], "flop": 2.0 * T * H * N,
                "flag_driven_us": timed(lambda: FL.ag_gemm(slot, g, x, slot.stage, dy, mg, H, N, T, 1, 1, 2, 1, False, False, False)),
                "flag_driven_err": err_ag,
                "plain_gemm_on_stage_us": timed(lambda: native.gemm(slot.stage, dy, trans_a=True, out=mg, accumulate=True)),
                "plain_gemm_on_stage_err": err_plain,
                "cublas_bf16_out_us": timed(lambda: torch.matmul(xfull.t(), dy))}
        emit(wrec)
        del slot

    for name, K in row_shapes.items():
        N = H
        a = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16)
        w = (torch.randn(K, N, device="cuda") * 0.05).to(torch.bfloat16)
        out = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
        ref = spu.reduce_scatter(torch.matmul(a, w).float(), g)
        rec = {"op": f"gemm_rs_{name}", "shape": [T, K, N],
               "cublas_us": timed(lambda: torch.matmul(a, w)),
               "plain_gemm_us": timed(lambda: native.gemm(a, w)),
               "nccl_rs_us": timed(lambda: spu.reduce_scatter(torch.matmul(a, w), g)) ,
               "compute_bound_us": 2.0 * T * K * N / 1644e12 * 1e6,
               "link_bound_us": (n - 1) * rows * N * 2 / 770e9 * 1e6}
        rec["unfused_us"] = rec.pop("nccl_rs_us")
        configs = [(False, 16)] + ([(True, 16)] if mc else [])
        if args.sweep and mc:
            configs += [(True, c) for c in (4, 8, 24, 32)]
        for use_mc, n_red in configs:
            pair = rs_pair(use_mc, n_red, N)
            state = {"i": 0}

            def run():
                s = pair[state["i"] & 1]
                state["i"] += 1
                FL.gemm_rs(s, g, a, w, out, T, N, K, 0, 1)
            out.zero_()
            run()
            torch.cuda.synchronize()
            err = rel(out, ref)
            t = timed(run)
            key = ("fused_nvls_red%d" % n_red) if use_mc else "fused_push"
            rec[key + "_us"] = t
            rec[key + "_err"] = err
            if args.trace and not use_mc:
                import ctypes

                import numpy as np
                k = _lib.kernels()
                k.pd_gemm_rs_trace(1)
                for _ in range(3):
                    run()
                torch.cuda.synchronize()
                tdist.barrier()
                buf = (ctypes.c_ulonglong * 2048)()
                k.pd_gemm_rs_trace_read(buf)
                k.pd_gemm_rs_trace(0)
                tt = np.array(list(buf), dtype=np.float64).reshape(256, 8)
                tt = tt[tt[:, 0] > 0]
                t0 = tt[:, 0].min()
                rec["trace_ctas"] = int(tt.shape[0])
                for nm, col in (("gemm_done", 1), ("signalled", 2), ("first_unit_ready", 4), ("first_unit_reduced", 5),
                                ("reduced", 3)):
                    v = (tt[:, col] - t0) / 1e3
                    v = v[v > 0]
                    if v.size:
                        rec[f"trace_{nm}_us"] = [round(float(v.min()), 1), round(float(np.median(v)), 1), round(float(v.max()), 1)]
            del pair
        emit(rec)
    if args.extra:
        _extra(args, g, n, rank, timed, rel, emit)
    tdist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


def _extra(args, g, n, rank, timed, rel, emit):
    """The other fused compute + collective kernels against their unfused sequences:
    decode GEMM -> all-reduce (13B row-parallel projections, 64 tokens), reduce-scatter (+ AdamW) of a gradient bucket,
    and the stage-3 linear (weight gather fused into forward / dgrad GEMMs, dW through GEMM -> reduce-scatter)."""
    import torch.distributed as tdist

    from paddle_b200.ops import native
    from paddle_b200.parallel.gemm_ar import GemmAllReduce
    from paddle_b200.parallel.rs_adamw import FusedRSAdamW
    from paddle_b200.parallel.zero3_linear import zero3_linear

    pg = g.process_group
    # ---- GEMM -> all-reduce, decode shapes of Llama-2 13B (hidden 5120, ffn 13824), batch 64
    M, Hd = 64, 5120
    for name, Kfull in (("out_proj", 5120), ("ffn2", 13824)):
        K = Kfull // n // 64 * 64
        x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(K, Hd, device="cuda") * 0.05).bfloat16()
        res = torch.randn(M, Hd, device="cuda").bfloat16()
        ref = x.float() @ w.float()
        tdist.all_reduce(ref, group=pg)
        ref = ref + res.float()
        rec = {"op": f"gemm_ar_{name}", "shape": [M, K, Hd], "bytes_weights": K * Hd * 2,
               "hbm_bound_us": K * Hd * 2 / 6546.6e3}
        forms = [("push", "0")] + ([("nvls", "1")] if n >= 2 else [])
        for form, env in forms:
            os.environ["PD_GEMM_AR_NVLS"] = env
            op = GemmAllReduce(g, Hd, m_cap=M)
            os.environ.pop("PD_GEMM_AR_NVLS")
            if form == "nvls" and not op.mc_recv:
                continue
            out = op(x, w, res)
            torch.cuda.synchronize()
            rec[f"fused_{form}_err"] = rel(out, ref)
            rec[f"fused_{form}_us"] = timed(lambda: op(x, w, res))

        def unfused():
            y = torch.matmul(x, w)
            tdist.all_reduce(y, group=pg)
            return y + res
        rec["unfused_us"] = timed(unfused)
        emit(rec)

    # ---- reduce-scatter of an fp32 gradient bucket (+ AdamW on the owned slice)
    shard = (64 << 20) // 4 // n                     # a 64 MB bucket
    grad = torch.randn(n * shard, device="cuda")
    outg = torch.empty(shard, device="cuda")
    master = torch.randn(shard, device="cuda")
    m_, v_ = torch.zeros(shard, device="cuda"), torch.zeros(shard, device="cuda")
    pshard = master.bfloat16()
    fused = FusedRSAdamW(g, shard)
    refg = torch.empty(shard, device="cuda")
    tdist.reduce_scatter_tensor(refg, grad, group=pg)
    fused.reduce(grad, outg)
    torch.cuda.synchronize()
    rec = {"op": "rs_bucket_64MB", "bytes": n * shard * 4, "link_bound_us": (n - 1) * shard * 4 / 770e3,
           "fused_reduce_err": rel(outg, refg), "fused_reduce_us": timed(lambda: fused.reduce(grad, outg)),
           "nccl_rs_us": timed(lambda: tdist.reduce_scatter_tensor(refg, grad, group=pg)),
           "fused_rs_adamw_us": timed(lambda: fused.step(grad, master, m_, v_, pshard, 1e-4, 0.9, 0.95, 1e-8, 0.01, 0.9, 0.95))}

    def unfused_opt():
        tdist.reduce_scatter_tensor(refg, grad, group=pg)
        native.adamw_flat(pshard, master, refg, m_, v_, 1e-4, 0.9, 0.95, 1e-8, 0.01, 0.9, 0.95)
    rec["nccl_rs_plus_adamw_us"] = timed(unfused_opt)
    emit(rec)

    # ---- stage-3 linear: tokens 4096, weight [4096, 12288] (7B qkv) stored as row slices
    T, K, N = args.tokens, args.hidden, 3 * args.hidden
    torch.manual_seed(11)
    w_full = (torch.randn(K, N, device="cuda") * 0.05).bfloat16()
    w_shard = w_full[rank * (K // n):(rank + 1) * (K // n)].clone().requires_grad_(True)
    x = (torch.randn(T, K, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    dy = (torch.randn(T, N, device="cuda") * 0.05).bfloat16()
    y = zero3_linear(x, w_shard, g)
    rec = {"op": "zero3_linear_qkv", "shape": [T, K, N], "fwd_err": rel(y, x.detach().float() @ w_full.float()),
           "flop_fwd": 2.0 * T * K * N, "gather_bytes": (n - 1) * (K // n) * N * 2}

    def fused_fb():
        yy = zero3_linear(x, w_shard, g)
        yy.backward(dy)
        x.grad = None
        w_shard.grad = None

    def unfused_fb():
        full = torch.empty(K, N, device="cuda", dtype=torch.bfloat16)
        tdist.all_gather_into_tensor(full, w_shard.detach(), group=pg)
        torch.matmul(x.detach(), full)
        full2 = torch.empty_like(full)
        tdist.all_gather_into_tensor(full2, w_shard.detach(), group=pg)            # stage 3 re-gathers for backward
        torch.matmul(dy, full2.t())
        dwf = torch.matmul(x.detach().t(), dy)
        dws = torch.empty(K // n, N, device="cuda", dtype=torch.bfloat16)
        tdist.reduce_scatter_tensor(dws, dwf, group=pg)
    with torch.no_grad():
        rec["fused_fwd_us"] = timed(lambda: zero3_linear(x.detach(), w_shard.detach(), g))

        def unfused_fwd():
            full = torch.empty(K, N, device="cuda", dtype=torch.bfloat16)
            tdist.all_gather_into_tensor(full, w_shard.detach(), group=pg)
            torch.matmul(x.detach(), full)
        rec["unfused_fwd_us"] = timed(unfused_fwd)
    rec["fused_fwd_bwd_us"] = timed(fused_fb)
    rec["unfused_fwd_bwd_us"] = timed(unfused_fb)
    rec["compute_bound_fwd_bwd_us"] = 3 * rec["flop_fwd"] / 1644e6
    emit(rec)


if __name__ == "__main__":
    main()
