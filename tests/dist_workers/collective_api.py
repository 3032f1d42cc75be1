"""Every collective on 2+ ranks; each rank dumps its results for the parent to compare with NumPy."""
import _common  # noqa: F401
import numpy as np
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist

dist.init_parallel_env()
rank, n = dist.get_rank(), dist.get_world_size()
dev = "cuda" if dist.get_backend() == "NCCL" else "cpu"
res = {}
x = paddle.to_tensor(np.arange(8, dtype=np.float32) + 10 * rank, place=dev)
t = x.clone(); dist.all_reduce(t); res["all_reduce_sum"] = t.numpy()
t = x.clone(); dist.all_reduce(t, dist.ReduceOp.MAX); res["all_reduce_max"] = t.numpy()
t = x.clone(); dist.all_reduce(t, dist.ReduceOp.AVG); res["all_reduce_avg"] = t.numpy()
t = x.clone(); dist.broadcast(t, 1); res["broadcast"] = t.numpy()
t = x.clone(); dist.reduce(t, 0); res["reduce"] = t.numpy()
lst = []; dist.all_gather(lst, x); res["all_gather"] = np.stack([a.numpy() for a in lst])
out = paddle.zeros([8 * n], place=dev) if False else paddle.to_tensor(np.zeros(8 * n, np.float32), place=dev)
dist.all_gather(out, x); res["all_gather_into"] = out.numpy()
rs = paddle.to_tensor(np.zeros(8 // n, np.float32), place=dev)
dist.reduce_scatter(rs, x); res["reduce_scatter"] = rs.numpy()
ins = [paddle.to_tensor(np.full(3, rank * 10 + j, np.float32), place=dev) for j in range(n)]
outs = []; dist.alltoall(outs, ins); res["alltoall"] = np.stack([o.numpy() for o in outs])
a2 = paddle.to_tensor(np.zeros(8, np.float32), place=dev)
dist.alltoall_single(a2, x); res["alltoall_single"] = a2.numpy()
sc = paddle.to_tensor(np.zeros(4, np.float32), place=dev)
dist.scatter(sc, [paddle.to_tensor(np.full(4, j + 1, np.float32), place=dev) for j in range(n)] if rank == 0 else None, 0)
res["scatter"] = sc.numpy()
if rank == 0:
    dist.send(x, 1)
elif rank == 1:
    r = paddle.to_tensor(np.zeros(8, np.float32), place=dev); dist.recv(r, 0); res["recv"] = r.numpy()
task = dist.stream.all_reduce(x.clone(), sync_op=False); task.wait(); res["async_ok"] = task.is_completed()
objs = []; dist.all_gather_object(objs, {"rank": rank}); res["objects"] = objs
g = dist.new_group(list(range(n)))
t = x.clone(); dist.all_reduce(t, group=g); res["group_all_reduce"] = t.numpy()
peer = (rank + 1) % n
rbuf = paddle.to_tensor(np.zeros(8, np.float32), place=dev)
tasks = dist.batch_isend_irecv([dist.P2POp(dist.isend, x, peer), dist.P2POp(dist.irecv, rbuf, (rank - 1) % n)])
[tk.wait() for tk in tasks]; res["batch_p2p"] = rbuf.numpy()
dist.barrier()
_common.dump(res)
