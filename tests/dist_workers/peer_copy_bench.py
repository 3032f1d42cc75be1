"""Bandwidth of the three device-to-peer copy paths (diagnostic)."""
import ctypes
import os

import _common
import torch

import paddle_b200 as paddle
import paddle_b200.distributed as dist
from paddle_b200.ops import _lib
from paddle_b200.parallel import symm

dist.init_parallel_env()
rank, n = dist.get_rank(), dist.get_world_size()
g = dist.collective._get_default_group()
nbytes = 64 << 20
blk = symm.SymmBlock(nbytes, g)
src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
peer = (rank + 1) % n
k = _lib.kernels()
res = {}
for target, name in ((blk.ptrs[peer], "peer"), (blk.ptrs[rank], "local")):
    for mode in (0, 1, 2):
        for nct in (4, 8, 16, 32, 64):
            def run():
                rc = k.pd_peer_copy(ctypes.c_void_p(target), ctypes.c_void_p(src.data_ptr()), ctypes.c_int64(nbytes),
                                    ctypes.c_int(mode), ctypes.c_int(nct), ctypes.c_void_p(_lib.status_buffer().data_ptr()),
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                assert rc == 0
            for _ in range(2):
                run()
            dist.barrier(); torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(5):
                run()
            e.record(); torch.cuda.synchronize()
            res[f"{name}_mode{mode}_ctas{nct}"] = nbytes / (s.elapsed_time(e) / 5 * 1e-3) / 1e9
dist.barrier(); torch.cuda.synchronize()
got = blk.local.clone()
_lib.check_status()
if rank == 0:
    for kk, v in res.items():
        print(f"{kk:28s} {v:8.1f} GB/s", flush=True)
_common.dump(res)
