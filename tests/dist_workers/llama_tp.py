"""Llama (tiny) under TP+SP vs its single-rank twin: same weights (sharded from the twin), same data;
dumps losses and gathered parameters after 3 steps.  argv: dtype, device-kind, policy."""
import os
import sys

import _common
import numpy as np
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200.distributed import fleet
from paddle_b200.models.llama import LlamaConfig, LlamaForCausalLM

dtype = sys.argv[1] if len(sys.argv) > 1 else "float32"
policy = sys.argv[2] if len(sys.argv) > 2 else "fused"
world = int(os.environ["PADDLE_TRAINERS_NUM"])
shard_deg = 2 if len(sys.argv) > 4 and sys.argv[4] == "sharding2" else 1      # mp x sharding (split parameters)
n = world // shard_deg
strategy = fleet.DistributedStrategy()
strategy.hybrid_configs = {"dp_degree": 1, "mp_degree": n, "sharding_degree": shard_deg,
                           "sharding_configs": {"split_param": shard_deg > 1, "comm_overlap": True,
                                                "comm_buffer_size_MB": 0.25}}
fleet.init(is_collective=True, strategy=strategy)
paddle.set_kernel_policy(policy)
hcg0 = fleet.get_hybrid_communicate_group()
rank = hcg0.get_model_parallel_rank()
shard_rank = hcg0.get_sharding_parallel_rank()
kw = dict(hidden_size=256, intermediate_size=512, num_attention_heads=2, num_hidden_layers=2, vocab_size=1024,
          dtype=dtype)
if dtype == "bfloat16":
    kw.update(hidden_size=512, intermediate_size=1024, num_attention_heads=4)
if len(sys.argv) > 3:
    kw["intermediate_size"] = int(sys.argv[3])      # e.g. 2752: per-rank FFN width 1376 at 2 ranks, not a multiple of 64
paddle.seed(7)
twin = LlamaForCausalLM(LlamaConfig.tiny(**kw))
tp = LlamaForCausalLM(LlamaConfig.tiny(tensor_parallel_degree=n, sequence_parallel=True, **kw))


def shard(name, full):
    if "qkv_proj" in name:
        return torch.cat([c.chunk(n, 1)[rank] for c in full.chunk(3, 1)], 1)
    if "gate_up_proj" in name:
        return torch.cat([c.chunk(n, 1)[rank] for c in full.chunk(2, 1)], 1)
    if "o_proj" in name or "down_proj" in name or "embed_tokens" in name:
        return full.chunk(n, 0)[rank]
    if "lm_head" in name:
        return full.chunk(n, 1)[rank]
    return full


def unshard(name, parts):
    if "qkv_proj" in name:
        cs = [p.chunk(3, 1) for p in parts]
        return torch.cat([torch.cat([c[i] for c in cs], 1) for i in range(3)], 1)
    if "gate_up_proj" in name:
        cs = [p.chunk(2, 1) for p in parts]
        return torch.cat([torch.cat([c[i] for c in cs], 1) for i in range(2)], 1)
    if "o_proj" in name or "down_proj" in name or "embed_tokens" in name:
        return torch.cat(parts, 0)
    if "lm_head" in name:
        return torch.cat(parts, 1)
    return parts[0]


tsd = twin.state_dict()
with torch.no_grad():
    for k, p in tp.state_dict().items():
        p.copy_(shard(k, tsd[k]))
mp = dtype == "bfloat16"
if mp:
    from paddle_b200.distributed.fleet.utils.mix_precision_utils import enable_main_grad
    enable_main_grad(twin), enable_main_grad(tp)
opt_t = paddle.optimizer.AdamW(1e-3, parameters=twin.parameters(), grad_clip=paddle.nn.ClipGradByGlobalNorm(1.0),
                               multi_precision=mp)
opt_p = paddle.optimizer.AdamW(1e-3, parameters=tp.parameters(), grad_clip=paddle.nn.ClipGradByGlobalNorm(1.0),
                               multi_precision=mp)
from paddle_b200.distributed.fleet.utils.sequence_parallel_utils import register_sequence_parallel_allreduce_hooks
register_sequence_parallel_allreduce_hooks(tp, 1)
tp_model = fleet.distributed_model(tp)
opt_p = fleet.distributed_optimizer(opt_p)
gen = torch.Generator().manual_seed(3)
S = (128 if n <= 2 else 64 * n) if dtype == "bfloat16" else 64      # fused kernels need 128 tokens per rank
data = torch.randint(0, 1024, (3, 2, S + 1), generator=gen)
lt, lp = [], []
for step in range(3):
    ids = paddle.to_tensor(data[step].numpy())
    a = twin(ids[:, :-1], ids[:, 1:]); a.backward(); opt_t.step(); opt_t.clear_grad(); lt.append(float(a))
    if shard_deg > 1:          # the sharding ranks split the batch; the twin sees all of it
        ids = ids[shard_rank:shard_rank + 1]
    b = tp_model(ids[:, :-1], ids[:, 1:]); b.backward(); opt_p.step(); opt_p.clear_grad()
    if shard_deg > 1:
        t = torch.tensor([float(b)]); dist.all_reduce(t, group=hcg0.get_sharding_parallel_group()); b = float(t) / shard_deg
    lp.append(float(b))
g = fleet.get_hybrid_communicate_group().get_model_parallel_group()
maxdiff, diffs = 0.0, {}
for k, p in tp.state_dict().items():
    parts = []
    dist.all_gather(parts, p.detach().contiguous(), g)
    full = unshard(k, [x.float() for x in parts])
    diffs[k] = float((full - tsd[k].detach().float()).abs().max())
    maxdiff = max(maxdiff, diffs[k])
from paddle_b200.ops import native
extra = {}
if shard_deg > 1:
    # optimizer state written with gather=True has the reference's per-parameter keys and full tensors
    osd = opt_p.state_dict(gather=True)
    name = next(p.name for p in tp.parameters())
    extra = {"opt_keys_ok": all(f"{p.name}_moment1_0" in osd and f"{p.name}_moment2_0" in osd for p in tp.parameters()),
             "moment_shape_ok": all(tuple(osd[f"{p.name}_moment1_0"].shape) == tuple(p.shape) for p in tp.parameters()),
             "n_buckets": len(opt_p._inner_opt.__dict__["_buffers"])}
_common.dump({"twin": lt, "tp": lp, "maxdiff": maxdiff, "diffs": diffs, "launches": native.LAUNCH_COUNT, **extra})
