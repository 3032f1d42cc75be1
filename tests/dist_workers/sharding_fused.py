"""Fused sharding kernels on 2+ GPUs: (1) reduce-scatter + AdamW in one kernel against NCCL reduce_scatter + the
plain AdamW formula, several steps; (2) the stage-3 linear whose weight gather is fused into the GEMM, forward and
backward against the dense computation."""
import os

import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200.distributed import fleet
from paddle_b200.ops import _lib

n = int(os.environ["PADDLE_TRAINERS_NUM"])
strategy = fleet.DistributedStrategy()
strategy.hybrid_configs = {"dp_degree": 1, "mp_degree": 1, "sharding_degree": n}
fleet.init(is_collective=True, strategy=strategy)
rank = dist.get_rank()
g = fleet.get_hybrid_communicate_group().get_sharding_parallel_group()
from paddle_b200.parallel.rs_adamw import FusedRSAdamW
from paddle_b200.parallel.zero3_linear import zero3_linear

res = {}
shard = 100003                      # not a multiple of the chunk or of 4: exercises the tails
fused = FusedRSAdamW(g, shard)
torch.manual_seed(10 + rank)
master = torch.randn(shard, device="cuda")
m, v = torch.zeros(shard, device="cuda"), torch.zeros(shard, device="cuda")
param = master.bfloat16()
rm, rmm, rv = master.clone(), m.clone(), v.clone()
lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
errs, perr = [], []
for step in range(1, 4):
    grad = torch.randn(n * shard, device="cuda")
    scale = torch.tensor([1.0 / n], device="cuda")
    fused.step(grad, master, m, v, param, lr, b1, b2, eps, wd, b1 ** step, b2 ** step, grad_scale=scale)
    red = torch.empty(shard, device="cuda")
    dist.reduce_scatter(red, list(grad.chunk(n)), group=g)
    gg = red / n
    rm *= 1 - lr * wd
    rmm = b1 * rmm + (1 - b1) * gg
    rv = b2 * rv + (1 - b2) * gg * gg
    rm += -(lr / (1 - b1 ** step)) * rmm / (rv.sqrt() / (1 - b2 ** step) ** 0.5 + eps)
    errs.append(float((master - rm).abs().max()))
    # the bf16 copy may round a master value that sits on a rounding boundary the other way: allow one bf16 ulp there
    perr.append(float(((param.float() - rm.bfloat16().float()).abs() / rm.abs().clamp_min(1.0)).max()))
res["rs_adamw_err"] = max(errs)
res["rs_adamw_param_ulp_err"] = max(perr)
torch.cuda.synchronize()
_lib.check_status()

# ---- stage-3 linear with the gather fused into the GEMM
torch.manual_seed(3)                 # same full tensors on every rank
errs = []
# second shape: rows of 16400 bytes, wider than one 16 KB piece of the bulk-copy ring (a row then travels in segments)
for (K, N, M), reps in (((256 * n, 512, 384), 3), ((128 * n, 8200, 256), 2)):
  w_full = (torch.randn(K, N, device="cuda") * 0.05).bfloat16()
  x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16().requires_grad_(True)
  w_shard = w_full[rank * (K // n):(rank + 1) * (K // n)].clone().requires_grad_(True)
  for it in range(reps):
    y = zero3_linear(x, w_shard, g)
    dy = (torch.randn(M, N, device="cuda") * 0.1).bfloat16()
    y.backward(dy)
    ref = x.detach().float() @ w_full.float()
    errs.append(float((y.float() - ref).abs().max() / ref.abs().max()))
    rdx = dy.float() @ w_full.float().t()
    errs.append(float((x.grad.float() - rdx).abs().max() / rdx.abs().max()))
    rdw = (x.detach().float().t() @ dy.float()) * n          # every rank holds the same x, dy: the reduce sums n copies
    sl = rdw[rank * (K // n):(rank + 1) * (K // n)]
    errs.append(float((w_shard.grad.float() - sl).abs().max() / sl.abs().max()))
    x.grad = None
    w_shard.grad = None
res["zero3_linear_err"] = max(errs)
torch.cuda.synchronize()
_lib.check_status()

# ---- standalone symmetric-memory collectives against NCCL, eager and from a CUDA graph
from paddle_b200.parallel.symm_collectives import SymmCollectives
sc = SymmCollectives(g, 1 << 20)
errs = []
for dtype, numel in ((torch.float32, 1000), (torch.bfloat16, 70001 * 2), (torch.float32, 262144)):
    x = torch.randn(numel, device="cuda").to(dtype)
    ref = x.clone()
    dist.all_reduce(ref, group=g)
    errs.append(float((sc.all_reduce(x).float() - ref.float()).abs().max() / ref.float().abs().max()))
    gathered = sc.all_gather(x)
    parts = []
    dist.all_gather(parts, x, group=g)
    errs.append(float((gathered.float() - torch.cat([p.as_subclass(torch.Tensor) for p in parts]).float()).abs().max()))
    if numel % n == 0:
        rs_ref = torch.empty(numel // n, device="cuda", dtype=dtype)
        dist.reduce_scatter(rs_ref, list(x.chunk(n)), group=g)
        errs.append(float((sc.reduce_scatter(x).float() - rs_ref.float()).abs().max() / rs_ref.float().abs().max()))
for dtype, rows_each, width in ((torch.bfloat16, 5, 33), (torch.float32, 64, 1024), (torch.uint8, 3, 7)):
    x = (torch.randn(n * rows_each, width, device="cuda") * 40).to(dtype)
    a2a_ref = torch.empty_like(x)
    dist.alltoall_single(a2a_ref, x, group=g)
    errs.append(float((sc.all_to_all(x).float() - a2a_ref.as_subclass(torch.Tensor).float()).abs().max()))
res["symm_coll_err"] = max(errs)
# poisoned receive buffers: every byte a collective reads must have been written by a peer in THIS call, so filling
# both receive slots with NaN beforehand may not change any result (a read-before-arrival would surface as NaN)
poison_bad = 0
for it in range(4):
    dist.barrier(group=g)
    torch.cuda.synchronize()
    sc.block.local[:sc.off_cnt].view(torch.float32).fill_(float("nan"))
    torch.cuda.synchronize()
    dist.barrier(group=g)
    x = torch.randn(3 * 8192 + 100, device="cuda")
    ref = x.clone()
    dist.all_reduce(ref, group=g)
    got = sc.all_reduce(x)
    poison_bad += int(torch.isnan(got).any()) + int((got - ref).abs().max() > 1e-4 * ref.abs().max())
    gat = sc.all_gather(x)
    poison_bad += int(torch.isnan(gat).any())
res["symm_coll_poisoned_bad"] = poison_bad
# determinism: the reduction order is the rank order, so two runs on the same input agree bit for bit
xd = torch.randn(50000, device="cuda").bfloat16()
a1, a2 = sc.all_reduce(xd).clone(), sc.all_reduce(xd).clone()
r1, r2 = sc.reduce_scatter(xd).clone(), sc.reduce_scatter(xd).clone()
res["symm_coll_bitwise_repeatable"] = bool(torch.equal(a1, a2) and torch.equal(r1, r2))
xs = torch.randn(4096, device="cuda")
outg = torch.empty_like(xs)
side = torch.cuda.Stream()
side.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(side):
    sc.all_reduce(xs, out=outg)
torch.cuda.current_stream().wait_stream(side)
graph = torch.cuda.CUDAGraph()
with torch.cuda.graph(graph):
    sc.all_reduce(xs, out=outg)
ref = xs.clone()
dist.all_reduce(ref, group=g)
ge = []
for _ in range(3):
    outg.zero_()
    graph.replay()
    ge.append(float((outg - ref).abs().max()))
res["symm_coll_graph_err"] = max(ge)
torch.cuda.synchronize()
_lib.check_status()
# vocab-parallel cross entropy: the symmetric-memory exchange kernel against the two-all-reduce form, forward and
# backward, rows not a multiple of the block, ignored labels, two different row counts in turn
from paddle_b200.distributed.fleet.layers.mpu import mp_ops
ce_err = []
for rows in (1000, 4096, 1000):
    torch.manual_seed(77)                                   # same labels everywhere
    V = 512
    labels = torch.randint(0, V * n, (rows,), device="cuda")
    labels[::17] = -100
    torch.manual_seed(100 + rank)
    lg = torch.randn(rows, V, device="cuda").bfloat16()
    outs = []
    for fusedce in ("1", "0"):
        os.environ["PD_FUSED_CE"] = fusedce
        l = lg.clone().requires_grad_(True)
        loss = mp_ops._ParallelCE.apply(l, labels, g, -100)
        loss.sum().backward()
        outs.append((loss.detach().float(), l.grad.float()))
    os.environ.pop("PD_FUSED_CE")
    ce_err.append(float((outs[0][0] - outs[1][0]).abs().max()))
    ce_err.append(float((outs[0][1] - outs[1][1]).abs().max()))
res["fused_ce_err"] = max(ce_err)
torch.cuda.synchronize()
_lib.check_status()
# vocabulary-parallel embedding written straight into the sequence shards, against the plain lookup in the full table
emb_err = []
for T_tok in (n * 96, n * 1000):
    Vs, Hh = 256, 512
    torch.manual_seed(5)
    full_table = (torch.randn(n * Vs, Hh, device="cuda") * 0.5).bfloat16()
    ids = torch.randint(0, n * Vs, (T_tok,), device="cuda")
    wsh = full_table[rank * Vs:(rank + 1) * Vs].clone().requires_grad_(True)
    shard = mp_ops._VocabEmbedToSeqShard.apply(ids, wsh, g, rank * Vs)
    rows = T_tok // n
    ref_t = full_table.clone().float().requires_grad_(True)
    ref_full = torch.nn.functional.embedding(ids, ref_t)
    emb_err.append(float((shard.float() - ref_full[rank * rows:(rank + 1) * rows]).abs().max()))
    torch.manual_seed(6)
    dy_full = torch.randn(T_tok, Hh, device="cuda").bfloat16()
    shard.backward(dy_full[rank * rows:(rank + 1) * rows])
    ref_full.backward(dy_full.float())
    ref_dw = ref_t.grad[rank * Vs:(rank + 1) * Vs]
    emb_err.append(float((wsh.grad.float() - ref_dw).abs().max() / ref_dw.abs().max()))
res["fused_embedding_err"] = max(emb_err)
torch.cuda.synchronize()
_lib.check_status()
# in-switch (NVLS) two-shot all-reduce: sizes that change from call to call (the per-block arrival counts must carry
# over), a poisoned buffer, and CUDA-graph replay
res["symm_nvls"] = bool(sc.nvls_available())
if sc.nvls_available():
    ne = []
    for dtype, numel in ((torch.float32, 262144), (torch.bfloat16, 8 * 1000), (torch.bfloat16, 524288),
                         (torch.float32, 4 * 33333), (torch.bfloat16, 8 * 1000)):
        x = torch.randn(numel, device="cuda").to(dtype)
        ref = x.float().clone()
        dist.all_reduce(ref, group=g)
        dist.barrier(group=g)
        torch.cuda.synchronize()
        sc._nvls_state()["block"].local[: numel * x.element_size()].fill_(0xFF)   # NaN pattern in both dtypes
        torch.cuda.synchronize()
        dist.barrier(group=g)
        got = sc.all_reduce_nvls(x)
        ne.append(float((got.float() - ref).abs().max() / ref.abs().max()) if not torch.isnan(got.float()).any() else 1e9)
    res["symm_nvls_err"] = max(ne)
    xs = torch.randn(1 << 18, device="cuda").bfloat16()
    outg = torch.empty_like(xs)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        sc.all_reduce_nvls(xs, out=outg)
    torch.cuda.current_stream().wait_stream(side)
    graph2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph2):
        sc.all_reduce_nvls(xs, out=outg)
    ref = xs.float().clone()
    dist.all_reduce(ref, group=g)
    ge = []
    for _ in range(3):
        outg.zero_()
        graph2.replay()
        ge.append(float((outg.float() - ref).abs().max() / ref.abs().max()))
    res["symm_nvls_graph_err"] = max(ge)
    torch.cuda.synchronize()
    _lib.check_status()
_common.dump(res)
