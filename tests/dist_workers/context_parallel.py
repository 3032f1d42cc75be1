"""Ulysses and ring attention over a sequence split across 2 ranks vs plain attention on the whole sequence
(outputs and input gradients, causal and full, grouped-query heads for the ring form)."""
import math

import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200.distributed.fleet.meta_parallel.context_parallel import ring_attention, ulysses_attention

dist.init_parallel_env()
rank, n = dist.get_rank(), dist.get_world_size()
group = dist.new_group(list(range(n)))
B, S, Hq, Hk, D = 2, 8 * n, 4, 2, 8
g = torch.Generator().manual_seed(3)
q_full = torch.randn(B, S, Hq, D, generator=g)
k_full = torch.randn(B, S, Hk, D, generator=g)
v_full = torch.randn(B, S, Hk, D, generator=g)
w_full = torch.randn(B, S, Hq, D, generator=g)


def ref_attention(q, k, v, causal):
    q, k, v = q.clone().requires_grad_(), k.clone().requires_grad_(), v.clone().requires_grad_()
    kk, vv = k.repeat_interleave(Hq // Hk, 2), v.repeat_interleave(Hq // Hk, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) / math.sqrt(D)
    if causal:
        s = s.masked_fill(~torch.tril(torch.ones(S, S, dtype=torch.bool)), float("-inf"))
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vv)
    (o * w_full).sum().backward()
    return o.detach(), q.grad, k.grad, v.grad


def plain_attn(q, k, v, causal, scale):
    kk, vv = k.repeat_interleave(q.shape[2] // k.shape[2], 2), v.repeat_interleave(q.shape[2] // v.shape[2], 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) / math.sqrt(D)
    if causal:
        L = q.shape[1]
        s = s.masked_fill(~torch.tril(torch.ones(L, L, dtype=torch.bool)), float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vv)


sl = slice(rank * S // n, (rank + 1) * S // n)
res = {}
for causal in (False, True):
    ro, rq, rk, rv = ref_attention(q_full, k_full, v_full, causal)
    for name, fn in (("ring", lambda q, k, v: ring_attention(q, k, v, group, causal=causal)),
                     ("ulysses", lambda q, k, v: ulysses_attention(q, k, v, group, causal=causal, attn_fn=plain_attn))):
        q = q_full[:, sl].clone().requires_grad_(); k = k_full[:, sl].clone().requires_grad_()
        v = v_full[:, sl].clone().requires_grad_()
        o = torch.as_tensor(fn(q, k, v)).as_subclass(torch.Tensor)
        (o * w_full[:, sl]).sum().backward()
        key = f"{name}_{'causal' if causal else 'full'}"
        res[key] = max(float((o.detach() - ro[:, sl]).abs().max()), float((q.grad - rq[:, sl]).abs().max()),
                       float((k.grad - rk[:, sl]).abs().max()), float((v.grad - rv[:, sl]).abs().max()))
_common.dump(res)
