"""Python face of the native NCCL process group (``csrc/runtime/process_group.cc``).

``NativeProcessGroup`` brings up one communicator per group through the job's TCP store (rank 0 creates the NCCL unique
id, the others read it), issues collectives on the group's communication stream and returns ``Task`` objects with the
reference's semantics (``wait()`` = the compute stream waits for the result; ``wait(timeout)`` = the host blocks, bounded,
and learns about a communicator error or a timeout; python/paddle/distributed/communication/group.py, ProcessGroupNCCL in
paddle/fluid/distributed/collective/process_group_nccl.cc:899-993).  A timeout or an error report from a peer (published
under ``pd/comm_error/<group>`` in the store) aborts the communicator so that no rank stays blocked in a kernel.
The framework's default collectives run on ``torch.distributed``; this class is the native path for callers that need
their own communicators, streams and bounded waits (and it is what the fault tests drive with stand-in libraries)."""
from __future__ import annotations

import ctypes

import torch

_DTYPES = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
           torch.float64: 8, torch.bfloat16: 9}
_OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}
ALL_REDUCE, ALL_GATHER, REDUCE_SCATTER, BROADCAST, REDUCE, SEND, RECV = range(7)


class CommError(RuntimeError):
    """A collective did not finish: ``kind`` is ``"timeout"`` or ``"comm_error"``."""

    def __init__(self, kind, msg):
        super().__init__(msg)
        self.kind = kind


def _rt():
    from ..ops import _lib
    rt = _lib.runtime()
    rt.pd_pg_create.restype = ctypes.c_void_p
    rt.pd_pg_collective.restype = ctypes.c_int64
    return rt


def load(nccl_path=None, cudart_path=None):
    """Resolve NCCL and the CUDA runtime (default: the copies PyTorch has already loaded)."""
    rc = _rt().pd_pg_load(nccl_path.encode() if nccl_path else None, cudart_path.encode() if cudart_path else None)
    if rc != 0:
        raise RuntimeError({-1: "libnccl not found", -2: "libcudart not found", -3: "libnccl lacks a required symbol",
                            -4: "libcudart lacks a required symbol"}.get(rc, f"pd_pg_load failed ({rc})"))


class Task:
    def __init__(self, pg, tid, what):
        self._pg, self._id, self._what = pg, tid, what

    def is_completed(self):
        return bool(self._pg._rt.pd_pg_task_done(self._pg._h, ctypes.c_int64(self._id)))

    def wait(self, timeout=None):
        """``timeout=None``: make the current compute stream wait for the result (returns at once on the host).
        ``timeout`` in seconds: block the host; raises :class:`CommError` on a timeout or a communicator error and
        aborts the group (after telling the peers through the store) so that nothing stays blocked on the device."""
        pg = self._pg
        ms = -1 if timeout is None else int(timeout * 1000)
        rc = pg._rt.pd_pg_task_wait(pg._h, ctypes.c_int64(self._id), ms, pg._calc_stream())
        if rc == 0:
            return True
        kind = {1: "timeout", 2: "comm_error"}.get(rc)
        if kind is None:
            raise RuntimeError(f"waiting for {self._what} failed ({rc})")
        pg.report_error(f"{kind} in {self._what} on rank {pg.rank}")
        pg.abort()
        raise CommError(kind, f"{self._what} on group {pg.name!r} rank {pg.rank}: {kind}")


class NativeProcessGroup:
    def __init__(self, rank, nranks, device=0, store=None, name="default", unique_id=None):
        self._rt = _rt()
        self.rank, self.nranks, self.device, self.name, self._store = rank, nranks, device, name, store
        if unique_id is None:
            key = f"pd/nccl_id/{name}"
            if rank == 0:
                buf = ctypes.create_string_buffer(128)
                if self._rt.pd_pg_unique_id(buf) != 0:
                    raise RuntimeError("ncclGetUniqueId failed (call native_pg.load() first)")
                unique_id = buf.raw
                if store is not None:
                    store.set(key, unique_id)
            else:
                unique_id = bytes(store.get(key))
        self._h = ctypes.c_void_p(self._rt.pd_pg_create(unique_id, rank, nranks, device))
        if not self._h:
            raise RuntimeError("communicator bring-up failed")
        self.aborted = False

    def _calc_stream(self):
        if torch.cuda.is_available():
            return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return ctypes.c_void_p(0)

    def _call(self, kind, send, recv, count, dtype, op="sum", peer=0, sync_op=True, use_calc_stream=False, what=""):
        if self.aborted:
            raise CommError("comm_error", f"group {self.name!r} was aborted")
        self.check_peer_errors()
        nrc = ctypes.c_int(0)
        tid = self._rt.pd_pg_collective(
            self._h, kind, ctypes.c_void_p(send.data_ptr() if send is not None else 0),
            ctypes.c_void_p(recv.data_ptr() if recv is not None else 0), ctypes.c_int64(count), _DTYPES[dtype], _OPS[op],
            peer, self._calc_stream(), 1 if use_calc_stream else 0, ctypes.byref(nrc))
        if tid < 0:
            raise CommError("comm_error", f"{what} could not be issued (code {tid}, nccl result {nrc.value})")
        task = Task(self, tid, what)
        if sync_op and not use_calc_stream:
            task.wait()
        return task

    # ---- collectives (tensors are contiguous; outputs allocated by the caller)
    def all_reduce(self, t, op="sum", sync_op=True, use_calc_stream=False):
        return self._call(ALL_REDUCE, t, t, t.numel(), t.dtype, op, 0, sync_op, use_calc_stream, "all_reduce")

    def all_gather(self, out, t, sync_op=True, use_calc_stream=False):
        return self._call(ALL_GATHER, t, out, t.numel(), t.dtype, "sum", 0, sync_op, use_calc_stream, "all_gather")

    def reduce_scatter(self, out, t, op="sum", sync_op=True, use_calc_stream=False):
        return self._call(REDUCE_SCATTER, t, out, out.numel(), t.dtype, op, 0, sync_op, use_calc_stream, "reduce_scatter")

    def broadcast(self, t, src, sync_op=True, use_calc_stream=False):
        return self._call(BROADCAST, t, t, t.numel(), t.dtype, "sum", src, sync_op, use_calc_stream, "broadcast")

    def reduce(self, t, dst, op="sum", sync_op=True, use_calc_stream=False):
        return self._call(REDUCE, t, t, t.numel(), t.dtype, op, dst, sync_op, use_calc_stream, "reduce")

    def send(self, t, dst, sync_op=True, use_calc_stream=False):
        return self._call(SEND, t, None, t.numel(), t.dtype, "sum", dst, sync_op, use_calc_stream, "send")

    def recv(self, t, src, sync_op=True, use_calc_stream=False):
        return self._call(RECV, None, t, t.numel(), t.dtype, "sum", src, sync_op, use_calc_stream, "recv")

    # ---- failure handling
    def report_error(self, text):
        """Publish this rank's failure so that the other ranks abort instead of waiting for it."""
        if self._store is not None:
            try:
                self._store.set(f"pd/comm_error/{self.name}", text.encode())
            except Exception:  # noqa: BLE001 - the store may be the thing that failed
                pass

    def check_peer_errors(self):
        """Abort and raise when another rank has reported a failure on this group."""
        if self._store is None or not hasattr(self._store, "check"):
            return
        key = f"pd/comm_error/{self.name}"
        try:
            seen = self._store.check([key]) if callable(getattr(self._store, "check", None)) else False
        except Exception:  # noqa: BLE001
            return
        if seen:
            msg = bytes(self._store.get(key)).decode(errors="replace")
            self.abort()
            raise CommError("comm_error", f"a peer reported a failure on group {self.name!r}: {msg}")

    def async_error(self):
        return self._rt.pd_pg_async_error(self._h) == 1

    def inflight(self):
        return self._rt.pd_pg_inflight(self._h)

    def abort(self):
        if not self.aborted:
            self._rt.pd_pg_abort(self._h)
            self.aborted = True

    def destroy(self):
        if self._h:
            self._rt.pd_pg_destroy(self._h)
            self._h = ctypes.c_void_p(0)
