"""``fleet.util`` helpers (python/paddle/distributed/fleet/base/util_factory.py ``UtilBase``): small collectives
over python values and file sharding across workers."""
from __future__ import annotations

import numpy as np
import torch


class UtilBase:
    def __init__(self):
        self.role_maker = None
        self.dist_strategy = None

    def _set_strategy(self, dist_strategy):
        self.dist_strategy = dist_strategy

    def _set_role_maker(self, role_maker):
        self.role_maker = role_maker

    @staticmethod
    def _dist():
        import torch.distributed as tdist
        return tdist if tdist.is_available() and tdist.is_initialized() else None

    def _rank_world(self):
        d = self._dist()
        if d is not None:
            return d.get_rank(), d.get_world_size()
        if self.role_maker is not None:
            return self.role_maker._worker_index(), self.role_maker._worker_num()
        return 0, 1

    def all_reduce(self, input, mode="sum", comm_world="worker"):
        arr = np.asarray(input)
        d = self._dist()
        if d is None:
            return arr
        t = torch.as_tensor(arr.astype(np.float64) if arr.dtype.kind == "f" else arr)
        if d.get_backend() == "nccl":
            t = t.cuda()
        op = {"sum": d.ReduceOp.SUM, "min": d.ReduceOp.MIN, "max": d.ReduceOp.MAX}[mode]
        d.all_reduce(t, op=op)
        return t.cpu().numpy().astype(arr.dtype)

    def barrier(self, comm_world="worker"):
        d = self._dist()
        if d is not None:
            d.barrier()

    def all_gather(self, input, comm_world="worker"):
        d = self._dist()
        if d is None:
            return [input]
        out = [None] * d.get_world_size()
        d.all_gather_object(out, input)
        return out

    def get_file_shard(self, files):
        """Contiguous split of ``files`` over the workers; the first ``len % n`` workers get one more."""
        if not isinstance(files, list):
            raise TypeError("files should be a list of file need to be read.")
        rank, n = self._rank_world()
        base, rem = divmod(len(files), n)
        begin = rank * base + min(rank, rem)
        return files[begin:begin + base + (1 if rank < rem else 0)]

    get_heter_file_shard = get_file_shard

    def print_on_rank(self, message, rank_id):
        if self._rank_world()[0] == rank_id:
            print(message)
