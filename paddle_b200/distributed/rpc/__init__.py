"""``paddle.distributed.rpc``: run Python callables on named workers (python/paddle/distributed/rpc/rpc.py).

The reference runs a brpc service per worker and discovers peers through a TCPStore on ``master_endpoint``.  Here
each worker runs a listener thread (authenticated ``multiprocessing.connection``), publishes its endpoint in a
``torch.distributed.TCPStore`` hosted by rank 0, and ``rpc_sync`` / ``rpc_async`` send a pickled
``(fn, args, kwargs)`` to the target and return the result (exceptions raised remotely are re-raised locally).
``shutdown`` is a barrier over the store followed by closing the listener, as in the reference."""
from __future__ import annotations

import collections
import concurrent.futures as _fut
import datetime
import os
import pickle
import socket
import threading
from multiprocessing.connection import Client, Listener

__all__ = ["init_rpc", "shutdown", "rpc_async", "rpc_sync", "get_worker_info", "get_all_worker_infos",
           "get_current_worker_info"]

WorkerInfo = collections.namedtuple("WorkerInfo", ["name", "rank", "ip", "port"])
_AUTH = b"paddle-b200-rpc"
_DEFAULT_TIMEOUT_MS = -1


class _State:
    store = None
    listener = None
    thread = None
    me = None
    workers = {}
    pool = None
    world = 0
    stopping = False


_S = _State()


def _serve(listener):
    while True:
        try:
            conn = listener.accept()
        except (OSError, EOFError):
            return
        threading.Thread(target=_handle, args=(conn,), daemon=True).start()


def _handle(conn):
    try:
        while True:
            try:
                msg = conn.recv_bytes()
            except (EOFError, OSError):
                return
            try:
                fn, args, kwargs = pickle.loads(msg)
                if fn is None:
                    conn.send_bytes(pickle.dumps((True, None)))
                    return
                reply = (True, fn(*args, **(kwargs or {})))
            except BaseException as e:          # delivered to the caller
                reply = (False, e)
            try:
                conn.send_bytes(pickle.dumps(reply))
            except Exception as e:
                conn.send_bytes(pickle.dumps((False, RuntimeError(f"rpc result is not picklable: {e}"))))
    finally:
        conn.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def init_rpc(name, rank=None, world_size=None, master_endpoint=None):
    import torch.distributed as tdist
    rank = int(os.environ["PADDLE_TRAINER_ID"]) if rank is None else rank
    world_size = int(os.environ["PADDLE_TRAINERS_NUM"]) if world_size is None else world_size
    master_endpoint = master_endpoint or os.environ["PADDLE_MASTER_ENDPOINT"]
    ep = os.environ.get("PADDLE_WORKER_ENDPOINT")
    ip, port = ep.rsplit(":", 1) if ep else ("127.0.0.1", _free_port())
    _S.listener = Listener((ip, int(port)), authkey=_AUTH)
    _S.thread = threading.Thread(target=_serve, args=(_S.listener,), daemon=True)
    _S.thread.start()
    mip, mport = master_endpoint.rsplit(":", 1)
    _S.store = tdist.TCPStore(mip, int(mport), world_size, rank == 0, timeout=datetime.timedelta(seconds=300))
    _S.me = WorkerInfo(name, rank, ip, int(port))
    _S.world = world_size
    _S.store.set(f"rpc/worker/{rank}", pickle.dumps(tuple(_S.me)))
    _S.workers = {}
    for r in range(world_size):
        info = WorkerInfo(*pickle.loads(_S.store.get(f"rpc/worker/{r}")))
        if info.name in _S.workers:
            raise RuntimeError(f"duplicate rpc worker name {info.name!r}")
        _S.workers[info.name] = info
    _S.pool = _fut.ThreadPoolExecutor(max_workers=8)
    _S.stopping = False


def _invoke(to, fn, args, kwargs, timeout):
    info = get_worker_info(to)
    conn = Client((info.ip, info.port), authkey=_AUTH)
    try:
        conn.send_bytes(pickle.dumps((fn, tuple(args or ()), dict(kwargs or {}))))
        if timeout is not None and timeout > 0 and not conn.poll(timeout / 1000.0):
            raise TimeoutError(f"rpc to {to!r} timed out after {timeout} ms")
        ok, val = pickle.loads(conn.recv_bytes())
    finally:
        conn.close()
    if not ok:
        raise val
    return val


class FutureWrapper:
    def __init__(self, fut):
        self._f = fut

    def wait(self, timeout=None):
        return self._f.result(timeout)

    def done(self):
        return self._f.done()


def rpc_sync(to, fn, args=None, kwargs=None, timeout=_DEFAULT_TIMEOUT_MS):
    return _invoke(to, fn, args, kwargs, timeout)


def rpc_async(to, fn, args=None, kwargs=None, timeout=_DEFAULT_TIMEOUT_MS):
    return FutureWrapper(_S.pool.submit(_invoke, to, fn, args, kwargs, timeout))


def shutdown():
    if _S.store is None:
        return
    # every worker must have finished issuing calls before any listener closes
    n = _S.store.add("rpc/shutdown", 1)
    import time
    t0 = time.time()
    while n < _S.world and time.time() - t0 < 300:
        time.sleep(0.01)
        n = _S.store.add("rpc/shutdown", 0)
    _S.pool.shutdown(wait=True)
    _S.listener.close()
    if _S.me.rank == 0:
        # the store lives in rank 0: keep it until every worker has seen the full count
        _S.store.add("rpc/left", 1)
        while _S.store.add("rpc/left", 0) < _S.world and time.time() - t0 < 300:
            time.sleep(0.01)
    else:
        _S.store.add("rpc/left", 1)
    _S.store = None
    _S.workers = {}


def get_worker_info(name):
    return _S.workers[name]


def get_all_worker_infos():
    return sorted(_S.workers.values(), key=lambda w: w.rank)


def get_current_worker_info():
    return _S.me
