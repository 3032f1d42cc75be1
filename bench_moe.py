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


class _Only:
    """A view of some parameters with the ``parameters()`` method that ``enable_main_grad`` walks."""

    def __init__(self, params):
        self._p = list(params)

    def parameters(self):
        return self._p


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
    ap.add_argument("--nccl-exchange", action="store_true",
                    help="comparison arm: dispatch / combine through NCCL all-to-all (global_scatter / global_gather) instead "
                         "of the fused fp8 exchange over peer memory")
    ap.add_argument("--no-dense-sharding", dest="dense_sharding", action="store_false",
                    help="replicate the optimizer state of the dense parameters and all-reduce their gradients")
    args = ap.parse_args()
    if args.nccl_exchange:
        os.environ["PD_FUSED_MOE"] = "0"

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
    shared = [p for p in model.parameters() if not getattr(p, "is_moe_param", False)]
    expert_params = [p for p in model.parameters() if getattr(p, "is_moe_param", False)]
    mk = lambda ps: paddle.optimizer.AdamW(learning_rate=1e-5, beta1=0.9, beta2=0.95, epsilon=1e-8, weight_decay=0.1,   # noqa: E731
                                           parameters=ps, multi_precision=True)
    dense_opt = None
    if world > 1 and args.dense_sharding:
        # expert parallel + sharding stage 1 for the dense (attention / router / embedding) parameters: they are
        # replicated, so their optimizer state is split over the ranks and their gradients are reduce-scattered
        # bucket by bucket under backward (split-parameter sharding optimizer); the experts are local to a rank
        from paddle_b200.distributed.fleet.meta_optimizers.dygraph_optimizer.dygraph_sharding_optimizer import (
            DygraphShardingOptimizerV2)

        class _ShardingTopology:
            def get_sharding_parallel_group(self): return group
            def get_sharding_parallel_world_size(self): return world
            def get_sharding_parallel_rank(self): return rank
            def get_model_parallel_group(self): return None
            def get_pipe_parallel_group(self): return None
        enable_main_grad(_Only(expert_params))
        dense_opt = DygraphShardingOptimizerV2(mk(shared), _ShardingTopology(),
                                               {"comm_overlap": True, "comm_buffer_size_MB": 256,
                                                "accumulate_steps": args.micro_batches})
        opt = mk(expert_params)
    else:
        enable_main_grad(model)
        opt = mk(model.parameters())
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
        if dense_opt is not None:
            dense_opt.step()
            dense_opt.clear_grad()
        elif world > 1:                                 # attention / router / embedding weights are replicated
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
                       "parallelism": f"ep{world}" + ("+sharding1(dense)" if dense_opt is not None else ""),
                       "exchange": "nccl all-to-all" if args.nccl_exchange else "fused fp8 dispatch / combine over peer memory",
                       "l2": "inputs larger than L2"}}))
    if world > 1:
        torch.cuda.synchronize()
        tdist.barrier()
        from paddle_b200.parallel import moe_exchange, symm
        moe_exchange._exchanges.clear()
        symm.release_all()
        tdist.barrier()
        tdist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
