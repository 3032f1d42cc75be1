"""Operators dispatched through the SPMD rule registry on a 2-rank mesh: each result's placement and its values
(after gathering) against the dense computation, plus gradients through a concat / split / attention chain."""
import _common
import numpy as np
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200.distributed import ProcessMesh, Replicate, Shard

dist.init_parallel_env()
rank, n = dist.get_rank(), dist.get_world_size()
mesh = ProcessMesh(list(range(n)), dim_names=["x"])
res = {}
g = torch.Generator().manual_seed(0)


def sh(t, pl, grad=False):
    return dist.shard_tensor(paddle.to_tensor(t.detach().numpy()), mesh, pl, stop_gradient=not grad)


def full(t):
    return dist.unshard_dtensor(t).numpy()


def check(key, out, want, placement=None):
    ok = np.allclose(full(out), want.numpy(), atol=1e-5)
    if placement is not None:
        ok = ok and repr(out.placements) == placement
    res[key] = ok if ok else (repr(out.placements), float(np.abs(full(out) - want.numpy()).max()) if full(out).shape == tuple(want.shape) else "shape")


a, b = torch.randn(4, 6, generator=g), torch.randn(4, 6, generator=g)
da, db = sh(a, [Shard(0)]), sh(b, [Shard(0)])
check("concat_other_dim", paddle.concat([da, db], axis=1), torch.cat([a, b], 1), "[Shard(dim=0)]")
check("concat_sharded_dim", paddle.concat([da, db], axis=0), torch.cat([a, b], 0), "[Replicate()]")
check("concat_mixed", paddle.concat([da, sh(b, [Replicate()])], axis=1), torch.cat([a, b], 1), "[Shard(dim=0)]")
check("stack", paddle.stack([da, db], axis=0), torch.stack([a, b], 0), "[Shard(dim=1)]")
parts = paddle.split(da, 3, axis=1)
res["split_n"] = len(parts)
check("split", parts[1], a.split(2, 1)[1], "[Shard(dim=0)]")
parts = paddle.split(sh(a, [Shard(1)]), 2, axis=1)
check("split_sharded_dim", parts[0], a.split(3, 1)[0], "[Replicate()]")
check("chunk", paddle.chunk(da, 2, axis=1)[1], a.chunk(2, 1)[1], "[Shard(dim=0)]")
ub = paddle.unbind(sh(a, [Shard(1)]), axis=0)
check("unbind", ub[2], a[2], "[Shard(dim=0)]")
check("unsqueeze", paddle.unsqueeze(da, 0), a.unsqueeze(0), "[Shard(dim=1)]")
check("squeeze", paddle.squeeze(paddle.unsqueeze(da, 1), 1), a, "[Shard(dim=0)]")
check("cumsum_free", paddle.cumsum(da, axis=1), a.cumsum(1), "[Shard(dim=0)]")
check("cumsum_sharded", paddle.cumsum(da, axis=0), a.cumsum(0), "[Replicate()]")
check("argmax", paddle.argmax(da, axis=1), a.argmax(1), "[Shard(dim=0)]")
check("max_dim", paddle.max(da, axis=1), a.max(1).values, "[Shard(dim=0)]")
t3 = torch.randn(2, 4, 4, generator=g)
check("triu", paddle.triu(sh(t3, [Shard(0)])), t3.triu(), "[Shard(dim=0)]")
check("triu_gather", paddle.triu(sh(t3, [Shard(1)])), t3.triu(), "[Replicate()]")
check("tile", paddle.tile(da, [1, 2]), a.repeat(1, 2), "[Shard(dim=0)]")
check("expand", paddle.expand(sh(a[:, :1].contiguous(), [Shard(0)]), [4, 5]), a[:, :1].expand(4, 5), "[Shard(dim=0)]")
lab = torch.tensor([0, 2, 1, 2])
check("one_hot", paddle.nn.functional.one_hot(sh(lab, [Shard(0)]), 3), torch.nn.functional.one_hot(lab, 3).float(), "[Shard(dim=0)]")
idx = torch.tensor([3, 0, 3])
check("index_select", paddle.index_select(sh(a, [Shard(1)]), paddle.to_tensor(idx.numpy()), axis=0), a.index_select(0, idx), "[Shard(dim=1)]")
check("pad", paddle.nn.functional.pad(da, [1, 2], value=0.5), torch.nn.functional.pad(a, [1, 2], value=0.5), "[Shard(dim=0)]")

# attention with heads split, gradients through concat / split
q, k, v = (torch.randn(2, 4, 8, 16, generator=g, requires_grad=True) for _ in range(3))       # [b, heads, s, d]
ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
(ref ** 2).sum().backward()
dq, dk, dv = (sh(t, [Shard(1)], grad=True) for t in (q, k, v))
out = torch.nn.functional.scaled_dot_product_attention(dq, dk, dv, is_causal=True)
res["sdpa_placement"] = repr(out.placements)
res["sdpa"] = bool(np.allclose(full(out), ref.detach().numpy(), atol=1e-5))
(out * out).sum().backward()
res["sdpa_dq"] = bool(np.allclose(dq.grad.numpy(), q.grad.chunk(n, 1)[rank].numpy(), atol=1e-5))
x1 = torch.randn(4, 6, generator=g, requires_grad=True)
x2 = torch.randn(4, 6, generator=g, requires_grad=True)
w = torch.randn(12, 4, generator=g, requires_grad=True)
h = torch.cat([x1, x2], 1) @ w
l1, l2 = h.split(2, 1)
ref = (l1 * torch.tanh(l2)).sum()
ref.backward()
d1, d2 = sh(x1, [Shard(0)], grad=True), sh(x2, [Shard(0)], grad=True)
dw = sh(w, [Replicate()], grad=True)
hh = paddle.matmul(paddle.concat([d1, d2], axis=1), dw)
p1, p2 = paddle.split(hh, 2, axis=1)
loss = (p1 * paddle.tanh(p2)).sum()
res["chain_loss"] = abs(float(dist.unshard_dtensor(loss)) - float(ref)) < 1e-4
loss.backward()
res["chain_dx"] = bool(np.allclose(d1.grad.numpy(), x1.grad.chunk(n, 0)[rank].numpy(), atol=1e-5))
res["chain_dw"] = bool(np.allclose(dw.grad.numpy(), w.grad.numpy(), atol=1e-4))
_common.dump(res)
