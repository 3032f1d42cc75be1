"""Stand-alone memory estimate for one configuration, usable as a script
(python/paddle/distributed/auto_tuner/memory_cost_model.py:18-140):

    python -m paddle_b200.distributed.auto_tuner.memory_cost_model --dp_degree 1 --mp_degree 8 --pp_degree 1 \
        --sharding_degree 1 --micro_batch_size 1 --num_layers 32 --hidden_size 4096 --num_attention_heads 32 \
        --vocab_size 32000 --seq_length 4096 --global_batch_size 16
"""
from __future__ import annotations

import argparse

from .cost_model import get_mem


def parse_arguments(argv=None):
    ap = argparse.ArgumentParser()
    for name, default in (("dp_degree", 1), ("mp_degree", 1), ("pp_degree", 1), ("vpp_degree", 1), ("sharding_degree", 1),
                          ("sharding_stage", 1), ("micro_batch_size", 1), ("hidden_size", 4096),
                          ("num_attention_heads", 32), ("num_layers", 32), ("seq_length", 4096), ("vocab_size", 32000),
                          ("global_batch_size", 16)):
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--use_recompute", type=lambda s: s.lower() in ("1", "true"), default=False)
    ap.add_argument("--recompute_granularity", default="full")
    return ap.parse_args(argv)


def get_model_memory_usage(args):
    """Bytes per GPU for the parsed arguments (or any object with the same attributes)."""
    cfg = {k: getattr(args, k) for k in ("dp_degree", "mp_degree", "pp_degree", "sharding_degree", "sharding_stage",
                                         "micro_batch_size", "use_recompute")}
    total = args.dp_degree * args.mp_degree * args.pp_degree * args.sharding_degree
    gb = get_mem(total, cfg, args.num_layers, args.hidden_size, args.num_attention_heads, args.vocab_size, args.seq_length,
                 args.global_batch_size)
    return gb * 2 ** 30


if __name__ == "__main__":
    print(f"memory usage: {get_model_memory_usage(parse_arguments()) / 2 ** 30:.2f} GB")
