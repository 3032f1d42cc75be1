"""Bus bandwidth and latency of the symmetric-memory collectives against NCCL, one process per GPU:

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m paddle_b200.parallel.bench_collectives

Sizes 4 KB .. 64 MB of bf16, device timing (CUDA events, max over ranks), CUDA-graph replay for the symmetric
kernels when ``--graph`` is given.  Prints one JSON line per (collective, size)."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as tdist


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    ms = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tdist.barrier()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    t = torch.tensor([sorted(ms)[len(ms) // 2]], device="cuda")
    tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--max-mb", type=int, default=64)
    ap.add_argument("--graph", action="store_true")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    import paddle_b200 as paddle
    from paddle_b200.distributed import collective as C
    from paddle_b200.parallel.symm_collectives import SymmCollectives
    paddle.set_device(f"gpu:{local}")
    paddle.distributed.init_parallel_env()
    g = C.get_group()
    n, rank = g.nranks, g.rank
    sc = SymmCollectives(g, args.max_mb << 20)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")      # larger than L2
    size = 4096
    while size <= (args.max_mb << 20):
        elems = size // 2
        x = torch.randn(elems, device="cuda").bfloat16()
        rows = torch.randn(n, elems // n, device="cuda").bfloat16()
        out_ar, out_ag = torch.empty_like(x), torch.empty(n * elems, device="cuda", dtype=torch.bfloat16)
        out_rs = torch.empty(elems // n, device="cuda", dtype=torch.bfloat16)
        cases = {
            # name: (ours, nccl, bytes on the bus per rank)
            "all_reduce": (lambda: sc._run(0, x, out_ar, size), lambda: tdist.all_reduce(out_ar), 2 * size * (n - 1) / n),
            "reduce_scatter": (lambda: sc.reduce_scatter(rows, out_rs),
                               lambda: tdist.reduce_scatter_tensor(out_rs, rows.reshape(-1)), size * (n - 1) / n),
        }
        if sc.nvls_available() and size >= 65536:
            cases["all_reduce_nvls"] = (lambda: sc.all_reduce_nvls(x, out_ar), lambda: tdist.all_reduce(out_ar),
                                        2 * size * (n - 1) / n)
        if size * n <= (args.max_mb << 20):
            cases["all_gather"] = (lambda: sc.all_gather(x, out_ag), lambda: tdist.all_gather_into_tensor(out_ag, x),
                                   size * (n - 1))
        for name, (ours, nccl, bus) in cases.items():
            fn = ours
            if args.graph:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    ours()
                torch.cuda.current_stream().wait_stream(side)
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    ours()
                fn = gr.replay
            t_ours = _time(fn, args.iters, flush if size >= (1 << 20) else None)
            t_nccl = _time(nccl, args.iters, flush if size >= (1 << 20) else None)
            if rank == 0:
                print(json.dumps({"op": name, "bytes": size, "n_gpus": n, "ours_us": t_ours * 1e3, "nccl_us": t_nccl * 1e3,
                                  "ours_busbw_gbs": bus / t_ours / 1e6, "nccl_busbw_gbs": bus / t_nccl / 1e6,
                                  "graph": args.graph}), flush=True)
        size *= 4
    from paddle_b200.ops import _lib
    torch.cuda.synchronize()
    _lib.check_status()
    tdist.barrier()
    tdist.destroy_process_group()


if __name__ == "__main__":
    main()
