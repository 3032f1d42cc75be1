"""``paddle.distributed.spawn`` (python/paddle/distributed/spawn.py:463): start ``nprocs`` processes running
``func(*args)`` with the launcher's environment contract."""
from __future__ import annotations

import multiprocessing as mp
import os
import socket
import sys
import traceback


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(func, args, rank, nprocs, eps, backend, err_q, env_extra):
    os.environ.update({"PADDLE_TRAINER_ID": str(rank), "PADDLE_TRAINERS_NUM": str(nprocs),
                       "PADDLE_TRAINER_ENDPOINTS": ",".join(eps), "PADDLE_CURRENT_ENDPOINT": eps[rank],
                       "PADDLE_MASTER": eps[0], "PADDLE_LOCAL_RANK": str(rank), "PADDLE_RANK_IN_NODE": str(rank),
                       "FLAGS_selected_gpus": str(rank)})
    if backend:
        os.environ["PADDLE_DISTRI_BACKEND"] = backend
    os.environ.update(env_extra or {})
    try:
        func(*args)
    except BaseException:  # noqa: BLE001
        err_q.put((rank, traceback.format_exc()))
        sys.exit(1)


class MultiprocessContext:
    def __init__(self, procs, err_q):
        self.processes, self._err_q = procs, err_q

    def join(self, timeout=None):
        for p in self.processes:
            p.join(timeout)
        failed = [p for p in self.processes if p.exitcode not in (0, None)]
        if failed:
            msg = ""
            while not self._err_q.empty():
                rank, tb = self._err_q.get()
                msg += f"\n----- process {rank} -----\n{tb}"
            for p in self.processes:
                if p.is_alive():
                    p.terminate()
            raise RuntimeError(f"{len(failed)} spawned process(es) failed:{msg}")
        return all(p.exitcode == 0 for p in self.processes)


def spawn(func, args=(), nprocs=-1, join=True, daemon=False, **options):
    if nprocs <= 0:
        import torch
        nprocs = max(torch.cuda.device_count(), 1)
    ctx = mp.get_context(options.get("start_method", "spawn"))
    base = _free_port()
    eps = [f"127.0.0.1:{base}"] + [f"127.0.0.1:{_free_port()}" for _ in range(nprocs - 1)]
    err_q = ctx.Queue()
    procs = []
    for r in range(nprocs):
        p = ctx.Process(target=_worker, args=(func, args, r, nprocs, eps, options.get("backend"), err_q,
                                              options.get("env")), daemon=daemon)
        p.start()
        procs.append(p)
    context = MultiprocessContext(procs, err_q)
    if join:
        context.join()
    return context
