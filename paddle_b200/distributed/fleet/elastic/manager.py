"""Elastic membership manager (python/paddle/distributed/fleet/elastic/manager.py:125 ``ElasticManager``).

Hosts register under ``/paddle/<job>/nodes/<host>`` with a time-to-live that a heartbeat thread keeps alive
(:254); every manager watches the node prefix (:237) and classifies membership changes against the allowed range
``np = MIN[:MAX]``: below MIN -> HOLD (wait for peers, fault-tolerance level) or EXIT after ``elastic_timeout``;
changed but within range -> RESTART with recomputed endpoints (scale-in/out, :484-560); trainers finished ->
COMPLETED.  The key-value service is pluggable: the reference talks to etcd, this module defines the small client
interface it needs and ships an in-memory implementation (tests, single host) and one over the framework's TCP
store (multi-host without etcd)."""
from __future__ import annotations

import os
import threading
import time

ELASTIC_EXIT_CODE = 101
ELASTIC_AUTO_PARALLEL_EXIT_CODE = 102
ELASTIC_TTL = 6


class ElasticLevel:
    FAULT_TOLERANCE = 1
    ELASTIC = 2


class ElasticStatus:
    COMPLETED = "completed"
    ERROR = "error"
    HOLD = "hold"
    RESTART = "restart"
    EXIT = "exit"


class MemoryKV:
    """In-process key-value service with leases and prefix watches (the subset of the etcd3 client used here)."""

    def __init__(self):
        self._d, self._ttl, self._watch = {}, {}, {}
        self._mu = threading.RLock()
        self._wid = 0

    class _Lease:
        def __init__(self, kv, ttl):
            self.kv, self.ttl, self.keys = kv, ttl, set()

        def refresh(self):
            with self.kv._mu:
                for k in self.keys:
                    if k in self.kv._d:
                        self.kv._ttl[k] = time.time() + self.ttl

        def revoke(self):
            for k in list(self.keys):
                self.kv.delete(k)

    def lease(self, ttl):
        return MemoryKV._Lease(self, ttl)

    def _expire(self):
        now = time.time()
        for k in [k for k, t in self._ttl.items() if t < now]:
            self.delete(k)

    def put(self, key, value, lease=None):
        with self._mu:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()
            if lease is not None:
                lease.keys.add(key)
                self._ttl[key] = time.time() + lease.ttl
            cbs = [cb for p, cb in self._watch.values() if key.startswith(p)]
        for cb in cbs:
            cb({"type": "put", "key": key})

    def get(self, key):
        with self._mu:
            self._expire()
            return self._d.get(key), None

    def get_prefix(self, prefix):
        with self._mu:
            self._expire()
            return [(v, k) for k, v in sorted(self._d.items()) if k.startswith(prefix)]

    def delete(self, key):
        with self._mu:
            existed = self._d.pop(key, None) is not None
            self._ttl.pop(key, None)
            cbs = [cb for p, cb in self._watch.values() if key.startswith(p)] if existed else []
        for cb in cbs:
            cb({"type": "delete", "key": key})

    def delete_prefix(self, prefix):
        for _, k in self.get_prefix(prefix):
            self.delete(k)

    def add_watch_prefix_callback(self, prefix, cb):
        with self._mu:
            self._wid += 1
            self._watch[self._wid] = (prefix, cb)
            return self._wid

    def cancel_watch(self, wid):
        with self._mu:
            self._watch.pop(wid, None)


class LauncherInterface:
    """What the manager needs from a launcher: start the local trainers, poll them, stop them."""

    def __init__(self, args):
        self.args = args
        self.procs = []

    def launch(self):
        pass

    def watch(self):
        """None while running, else the exit code."""
        return 0

    def stop(self):
        pass


class ElasticManager:
    def __init__(self, args, kv_client=None):
        self.args = args
        np_spec = str(getattr(args, "np", None) or getattr(args, "nnodes", "1"))
        lo, _, hi = np_spec.partition(":")
        self.min_np, self.max_np = int(lo), int(hi or lo)
        self.np = self.min_np
        self.job_id = getattr(args, "job_id", None) or os.getenv("PADDLE_ELASTIC_JOB_ID", "default")
        self.host = getattr(args, "host", None) or os.getenv("POD_IP", "127.0.0.1")
        self.elastic_timeout = int(getattr(args, "elastic_timeout", None) or os.getenv("PADDLE_ELASTIC_TIMEOUT", 30))
        self.elastic_level = int(getattr(args, "elastic_level", None) or
                                 (ElasticLevel.ELASTIC if self.max_np > self.min_np else ElasticLevel.FAULT_TOLERANCE))
        self.ttl = int(os.getenv("PADDLE_ELASTIC_TTL", ELASTIC_TTL))
        self.kv = kv_client if kv_client is not None else MemoryKV()
        self.enable = kv_client is not None or bool(getattr(args, "elastic_server", None))
        self.prefix = f"/paddle/{self.job_id}"
        self.node_prefix = f"{self.prefix}/nodes"
        self.np_path = f"{self.prefix}/np"
        self.endpoints_path = f"{self.prefix}/endpoints"
        self.host_path = f"{self.node_prefix}/{self.host}-{os.getpid()}-{id(self) & 0xffff}"
        self.hosts = []
        self.need_sync = False
        self.stopped = False
        self.launcher = None
        self.curr_host = f"{self.host}:{getattr(args, 'host_port', 6170)}"
        self.trainers = ""
        self._lease = self.kv.lease(self.ttl)
        self.kv.put(self.host_path, self.curr_host, lease=self._lease)
        self._hb = threading.Thread(target=self._heartbeat, daemon=True)
        self._hb.start()
        self._watch_id = self.kv.add_watch_prefix_callback(self.node_prefix, self._host_call_back)
        self.kv.put(self.np_path, str(self.np))

    # ------------------------------------------------------------------ membership
    def _heartbeat(self):
        while not self.stopped:
            try:
                self._lease.refresh()
                if self.kv.get(self.host_path)[0] is None:      # the lease ran out (pause, partition): re-register
                    self.kv.put(self.host_path, self.curr_host, lease=self._lease)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(max(self.ttl / 3.0, 0.05))

    def _host_call_back(self, event):
        self.hosts = [v.decode() for v, _ in self.kv.get_prefix(self.node_prefix)]
        self.need_sync = True

    def _completed(self):
        v, _ = self.kv.get(self.prefix)
        return v is not None and v.decode() == ElasticStatus.COMPLETED

    def _match(self, host_list=None):
        self.hosts = host_list if host_list is not None else \
            [v.decode() for v, _ in self.kv.get_prefix(self.node_prefix)]
        n = len(self.hosts)
        if self.elastic_level == ElasticLevel.FAULT_TOLERANCE:
            return n == self.np
        return self.min_np <= n <= self.max_np

    def _update_endpoints(self):
        """Scale-in / scale-out: keep surviving hosts in their old order, append newcomers."""
        old = [h for h in self.trainers.split(",") if h]
        keep = [h for h in old if h in self.hosts]
        new = keep + sorted(h for h in self.hosts if h not in keep)
        self.trainers = ",".join(new)
        self.np = len(new)
        self.kv.put(self.endpoints_path, self.trainers)
        self.kv.put(self.np_path, str(self.np))
        rank = new.index(self.curr_host) if self.curr_host in new else -1
        os.environ["PADDLE_TRAINERS"] = ",".join(h.split(":")[0] for h in new)
        os.environ["PADDLE_TRAINER_ENDPOINTS"] = self.trainers
        os.environ["PADDLE_TRAINER_ID"] = str(rank)
        os.environ["PADDLE_TRAINERS_NUM"] = str(self.np)
        return rank

    def wait(self):
        """Block until membership is acceptable (or the timeout runs out)."""
        if not self.enable:
            return True
        t0 = time.time()
        while not self.stopped:
            if self._match():
                self._update_endpoints()
                self.need_sync = False
                return True
            if time.time() - t0 > self.elastic_timeout:
                return False
            time.sleep(0.05)
        return False

    def run(self, launcher):
        self.launcher = launcher
        launcher.launch()

    def watch(self):
        """Poll trainers and membership; returns an ``ElasticStatus``."""
        if self.launcher is None:
            return ElasticStatus.ERROR
        hold_since = None
        while not self.stopped:
            ret = self.launcher.watch()
            if ret is not None:
                if ret == 0:
                    self.kv.put(self.prefix, ElasticStatus.COMPLETED)
                    return ElasticStatus.COMPLETED
                if ret in (ELASTIC_EXIT_CODE, ELASTIC_AUTO_PARALLEL_EXIT_CODE):
                    return ElasticStatus.RESTART
                return ElasticStatus.ERROR
            if self._completed():
                self.launcher.stop()
                return ElasticStatus.COMPLETED
            if self.need_sync:
                ok = self._match()
                if ok and set(self.hosts) != set(h for h in self.trainers.split(",") if h):
                    self.launcher.stop()
                    return ElasticStatus.RESTART
                if not ok:
                    hold_since = hold_since or time.time()
                    if len(self.hosts) < self.min_np or self.elastic_level == ElasticLevel.FAULT_TOLERANCE:
                        self.launcher.stop()
                        if time.time() - hold_since > self.elastic_timeout:
                            return ElasticStatus.EXIT
                        return ElasticStatus.HOLD
                else:
                    self.need_sync = False
            time.sleep(0.05)
        return ElasticStatus.EXIT

    def exit(self, completed=False):
        self.stopped = True
        if self.launcher is not None:
            self.launcher.stop()
        self.kv.cancel_watch(self._watch_id)
        if completed:
            self.kv.put(self.prefix, ElasticStatus.COMPLETED)
        self._lease.revoke()

    def signal_handler(self, sigint, frame):
        self.exit()
