"""Rendezvous key-value store backed by the native TCP store (``paddle_b200/csrc/runtime/tcp_store.cc``;
reference: paddle/phi/core/distributed/store/tcp_store.h:40-139)."""
from __future__ import annotations

import ctypes
import struct

from ..ops import _lib


class StoreTimeoutError(TimeoutError):
    pass


class TCPStore:
    def __init__(self, host="127.0.0.1", port=0, is_master=False, world_size=1, timeout=900):
        rt = _lib.runtime()
        rt.pd_store_create.restype = ctypes.c_void_p
        rt.pd_store_get.restype = ctypes.c_int64
        rt.pd_store_add.restype = ctypes.c_int64
        self._rt = rt
        self._h = rt.pd_store_create(host.encode(), int(port), 1 if is_master else 0, int(timeout * 1000))
        if not self._h:
            raise RuntimeError(f"cannot {'serve' if is_master else 'reach'} TCP store at {host}:{port}")
        self._h = ctypes.c_void_p(self._h)
        self.port = rt.pd_store_port(self._h)
        self.world_size = world_size

    def set(self, key, value):
        if isinstance(value, str):
            value = value.encode()
        if self._rt.pd_store_set(self._h, key.encode(), value, ctypes.c_int64(len(value))) != 0:
            raise RuntimeError("store set failed")

    def get(self, key):
        cap = 1 << 20
        buf = ctypes.create_string_buffer(cap)
        n = self._rt.pd_store_get(self._h, key.encode(), buf, ctypes.c_int64(cap))
        if n == -2:
            raise StoreTimeoutError(f"timed out waiting for key {key!r}")
        if n < 0:
            raise RuntimeError("store get failed")
        return buf.raw[:n]

    def add(self, key, amount=1):
        return int(self._rt.pd_store_add(self._h, key.encode(), ctypes.c_int64(amount)))

    def check(self, key):
        return self._rt.pd_store_check(self._h, key.encode()) == 1

    def delete_key(self, key):
        return self._rt.pd_store_delete(self._h, key.encode()) == 1

    def wait(self, key, timeout=None):
        rc = self._rt.pd_store_wait(self._h, key.encode(), int((timeout or 0) * 1000))
        if rc == -2:
            raise StoreTimeoutError(f"timed out waiting for key {key!r}")
        if rc != 0:
            raise RuntimeError("store wait failed")

    def barrier(self, name, world_size=None, timeout=None):
        n = world_size or self.world_size
        if self.add(f"{name}/count", 1) == n:
            self.set(f"{name}/done", b"1")
        self.wait(f"{name}/done", timeout)

    def close(self):
        if self._h:
            self._rt.pd_store_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
