"""Mixtral-style sparse-MoE training step: tokens/s with the experts as block-scaled fp8 grouped GEMMs
(``--experts grouped_fp8``) or as per-expert bf16 Linear layers (``--experts loop``, the reference's structure).

    python bench_moe.py --layers 4 --steps 3 --warmup 3
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench_moe.py --gpus 8 --layers 32

The layer shapes are Mixtral 8x7B's (hidden 4096, intermediate 14336, 8 experts, top-2, GQA 32/8).  With N > 1 ranks
the experts are spread over the ranks (expert parallel, all-to-all dispatch / combine) and every rank feeds its own
sequences.  ``--layers`` below 32 is a reduced-depth run (the JSON line says so): one GPU cannot hold the 32-layer
model with AdamW state.  Timing: CUDA events around ``--steps`` optimizer steps after ``--warmup`` steps, max over
ranks; inputs start in pinned host memory and the loss is read back every step."""
from __future__ import annotations

import argparse
import json
import os


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--micro-batches", type=int, default=4)
    ap.add_argument("--experts", default="grouped_fp8", choices=["grouped_fp8", "loop"])
    ap.add_argument("--model", default="mixtral-8x7b", choices=["mixtral-8x7b", "tiny"])
    args = ap.parse_args()

    import torch
    import torch.distributed as tdist

    import paddle_b200 as paddle
    from paddle_b200.models.mixtral import MixtralConfig, MixtralForCausalLM
    from paddle_b200.ops import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    paddle.set_device(f"gpu:{local_rank}")
    paddle.seed(1234 + rank)
    group = None
    if world > 1:
        import paddle_b200.distributed as dist
        dist.init_parallel_env()
        group = dist.new_group(list(range(world)))

    if args.model == "tiny":
        cfg = MixtralConfig.tiny(dtype="bfloat16", expert_impl=args.experts, max_position_embeddings=args.seq_len)
    else:
        cfg = MixtralConfig.mixtral_8x7b(num_hidden_layers=args.layers, dtype="bfloat16", expert_impl=args.experts,
                                         max_position_embeddings=args.seq_len)
    model = MixtralForCausalLM(cfg, moe_group=group)
    from paddle_b200.distributed.fleet.utils.mix_precision_utils import enable_main_grad
    enable_main_grad(model)
    opt = paddle.optimizer.AdamW(learning_rate=1e-5, beta1=0.9, beta2=0.95, epsilon=1e-8, weight_decay=0.1,
                                 parameters=model.parameters(), multi_precision=True)
    shared = [p for p in model.parameters() if not getattr(p, "is_moe_param", False)]
    seq, n_mb = args.seq_len, args.micro_batches
    gen = torch.Generator().manual_seed(4321 + rank)
    host_ids = torch.randint(0, cfg.vocab_size, (n_mb, 1, seq + 1), generator=gen, dtype=torch.int64).pin_memory()

    def train_step():
        total = None
        for i in range(n_mb):
            tok = host_ids[i].cuda(non_blocking=True)
            loss = model(tok[:, :-1], tok[:, 1:]) / n_mb
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if world > 1:                                   # attention / router / embedding weights are replicated
            for p in shared:
                g = getattr(p, "main_grad", None)
                g = g if g is not None else p.grad
                if g is not None:
                    tdist.all_reduce(g)
                    g.div_(world)
        opt.step()
        opt.clear_grad()
        return float(total)                             # device -> host read of the step's loss

    def barrier():
        if world > 1:
            tdist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        loss = train_step()
    barrier()
    l0 = native.LAUNCH_COUNT
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = train_step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
    if world > 1:
        tdist.all_reduce(ms, op=tdist.ReduceOp.MAX)
    ms = float(ms)
    tokens = world * n_mb * seq
    E, H, I, k = cfg.num_local_experts, cfg.hidden_size, cfg.intermediate_size, cfg.num_experts_per_tok
    expert_flops = 3 * 2 * (n_mb * seq * k) * 3 * H * I * cfg.num_hidden_layers          # fwd + dgrad + wgrad, per rank
    if rank == 0:
        launches = (native.LAUNCH_COUNT - l0) // max(args.steps, 1)
        print(json.dumps({
            "metric": "mixtral_moe_train_tokens_per_s", "value": tokens / ms * 1e3, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "dtype": "bf16 (experts fp8 e4m3 block-scaled)" if args.experts == "grouped_fp8" else "bf16",
            "data": "synthetic tokens from pinned host memory, random-init weights", "loss": loss,
            "expert_tflops_per_gpu": expert_flops / ms / 1e9, "gpu_launches_per_step": launches,
            "config": {"model": args.model, "layers": cfg.num_hidden_layers,
                       "reduced_depth": cfg.num_hidden_layers < 32 and args.model != "tiny",
                       "experts": args.experts, "global_batch": world * n_mb, "seq_len": seq,
                       "parallelism": f"ep{world}", "l2": "inputs larger than L2"}}))
    if world > 1:
        tdist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
