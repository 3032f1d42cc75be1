"""Serving benchmark: Llama-2 13B (random N(0, 0.02) weights), batch 64, prompt 1024 uniform random tokens, greedy
decode of 512 new tokens over a paged KV cache with 64-token pages, tensor parallel over N GPUs.

    python bench_decode.py                         # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench_decode.py --gpus N

Prints one JSON line: decode tokens/s (whole job), time to first token, both timed on the device with CUDA events
(max over ranks).  One untimed run warms up lazy initialisation and captures the decode CUDA graph."""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--model", default="llama2-13b", choices=["llama2-13b", "llama2-7b", "tiny"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--runs", type=int, default=1)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--nccl-ar", action="store_true", help="baseline: GEMM + NCCL all-reduce instead of the fused kernel")
    args = ap.parse_args()

    import torch
    import torch.distributed as tdist

    import paddle_b200 as paddle
    from paddle_b200.models.llama import LlamaConfig
    from paddle_b200.models.llama_infer import LlamaForCausalLMInference
    from paddle_b200.ops import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    paddle.set_device(f"gpu:{local_rank}")
    paddle.seed(1234)
    group = None
    if world > 1:
        from paddle_b200.distributed import fleet
        strategy = fleet.DistributedStrategy()
        strategy.hybrid_configs = {"dp_degree": 1, "mp_degree": world}
        fleet.init(is_collective=True, strategy=strategy)
        group = fleet.get_hybrid_communicate_group().get_model_parallel_group()
    cfg = {"llama2-13b": LlamaConfig.llama2_13b, "llama2-7b": LlamaConfig.llama2_7b,
           "tiny": lambda **kw: LlamaConfig.tiny(hidden_size=512, intermediate_size=1024, num_attention_heads=4,
                                                 num_hidden_layers=2, **kw)}[args.model](max_position_embeddings=4096)
    if args.nccl_ar:
        os.environ["PD_DECODE_NCCL_AR"] = "1"
    model = LlamaForCausalLMInference(cfg, tp_group=group)
    total = args.prompt + args.new_tokens
    model.prepare(max_batch=args.batch, max_seq_len=total)
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt), generator=gen).cuda()
    model.generate(ids, min(8, args.new_tokens), use_cuda_graph=not args.no_graph)       # warm-up + graph capture
    best = None
    for _ in range(args.runs):
        if world > 1:
            tdist.barrier()
        torch.cuda.synchronize()
        launches0 = native.LAUNCH_COUNT
        t = {}
        toks = model.generate(ids, args.new_tokens, use_cuda_graph=not args.no_graph, timings=t)
        vals = torch.tensor([t["ttft_ms"], t["decode_ms"]], device="cuda")
        if world > 1:
            tdist.all_reduce(vals, op=tdist.ReduceOp.MAX)
        ttft, dec = float(vals[0]), float(vals[1])
        if best is None or dec < best[1]:
            best = (ttft, dec, native.LAUNCH_COUNT - launches0)
    ttft, dec, launches = best
    steps = args.new_tokens - 1
    if rank == 0:
        print(json.dumps({
            "metric": "Llama-2 13B TP decode tok/s", "value": args.batch * steps / (dec / 1e3), "unit": "tokens/s",
            "n_gpus": world, "higher_is_better": True, "ttft_ms": ttft, "ms_per_decode_step": dec / steps,
            "prefill_tokens_per_s": args.batch * args.prompt / (ttft / 1e3), "dtype": "bf16",
            "data": "synthetic (uniform random prompt ids, N(0,0.02) random-init weights)", "vs_baseline": None,
            "config": {"model": args.model, "batch": args.batch, "prompt": args.prompt, "new_tokens": args.new_tokens,
                       "kv_cache": "paged, 64-token pages", "parallelism": f"tp{world}",
                       "cuda_graph": not args.no_graph,
                       "all_reduce": "nccl" if (args.nccl_ar or world == 1) else "fused into the GEMM kernel"},
            "kernel_launcher_calls_outside_graph": launches, "sample": toks[0, :8].tolist()}))
    if world > 1:
        tdist.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
