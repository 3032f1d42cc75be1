"""Job launcher: one process per GPU, environment contract, watch loop with restart
(python/paddle/distributed/launch/main.py:23 ``launch``; context/args_envs.py; controllers/collective.py:37-152
``build_pod``; controllers/controller.py:87-147 ``watch``; job/container.py:113 ``start``; controllers/master.py
``sync_peers``).

Single node needs no rendezvous.  With ``--nnodes > 1`` the node whose address is ``--master`` hosts a TCP store;
every node registers ``ip:free_ports`` there and reads the full endpoint list back (the reference does the same
through an HTTP or etcd master)."""
from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import time

ELASTIC_EXIT_CODE = 101


def _free_ports(n):
    socks, ports = [], []
    for _ in range(n):
        s = socket.socket()
        s.bind(("", 0))
        socks.append(s)
        ports.append(s.getsockname()[1])
    for s in socks:
        s.close()
    return ports


def parse_args(argv=None):
    env = os.environ
    p = argparse.ArgumentParser("paddle.distributed.launch")
    p.add_argument("--master", default=env.get("PADDLE_MASTER"), help="ip:port of the rendezvous store (multi-node)")
    p.add_argument("--nnodes", default=env.get("PADDLE_NNODES", "1"), help="N or MIN:MAX (elastic)")
    p.add_argument("--nproc_per_node", type=int, default=int(env["PADDLE_NPROC_PER_NODE"]) if env.get("PADDLE_NPROC_PER_NODE") else None)
    p.add_argument("--devices", "--gpus", dest="devices", default=env.get("PADDLE_DEVICES"))
    p.add_argument("--rank", type=int, default=int(env.get("PADDLE_RANK", -1)), help="node rank")
    p.add_argument("--log_dir", default=env.get("PADDLE_LOG_DIR", "log"))
    p.add_argument("--log_level", default=env.get("PADDLE_LOG_LEVEL", "INFO"))
    p.add_argument("--job_id", default=env.get("PADDLE_JOB_ID", "default"))
    p.add_argument("--run_mode", default=env.get("PADDLE_RUN_MODE", "collective"))
    p.add_argument("--max_restart", type=int, default=int(env.get("PADDLE_MAX_RESTART", 3)))
    p.add_argument("--elastic_level", type=int, default=int(env.get("PADDLE_ELASTIC_LEVEL", -1)))
    p.add_argument("--elastic_timeout", type=int, default=int(env.get("PADDLE_ELASTIC_TIMEOUT", 30)))
    p.add_argument("--host", default=env.get("POD_IP", "127.0.0.1"))
    p.add_argument("--backend", default=env.get("PADDLE_DISTRI_BACKEND"))
    p.add_argument("--poll_interval", type=float, default=0.5)
    p.add_argument("--auto_tuner_json", default=None, help="search hybrid-parallel configurations described by this JSON / YAML file")
    p.add_argument("training_script")
    p.add_argument("training_script_args", nargs=argparse.REMAINDER)
    return p.parse_args(argv)


class Container:
    """One rank process (launch/job/container.py)."""

    def __init__(self, entrypoint, env, log_file):
        self.entrypoint, self.env, self.log_file = entrypoint, env, log_file
        self.proc = None
        self._log = None

    def start(self):
        os.makedirs(os.path.dirname(self.log_file) or ".", exist_ok=True)
        self._log = open(self.log_file, "ab")
        self.proc = subprocess.Popen(self.entrypoint, env=self.env, stdout=self._log, stderr=subprocess.STDOUT,
                                     start_new_session=True)

    def poll(self):
        return None if self.proc is None else self.proc.poll()

    def terminate(self, grace=5.0):
        if self.proc is None or self.proc.poll() is not None:
            self._close()
            return
        try:
            os.killpg(self.proc.pid, signal.SIGTERM)     # the exact process group this container started
        except ProcessLookupError:
            pass
        t0 = time.time()
        while self.proc.poll() is None and time.time() - t0 < grace:
            time.sleep(0.05)
        if self.proc.poll() is None:
            try:
                os.killpg(self.proc.pid, signal.SIGKILL)
            except ProcessLookupError:
                pass
            self.proc.wait()
        self._close()

    def _close(self):
        if self._log is not None:
            self._log.close()
            self._log = None

    def tail(self, n=20):
        try:
            with open(self.log_file, "rb") as f:
                return b"\n".join(f.read().splitlines()[-n:]).decode(errors="replace")
        except OSError:
            return ""


class Pod:
    def __init__(self):
        self.containers = []

    def deploy(self):
        for c in self.containers:
            c.start()

    def stop(self):
        for c in self.containers:
            c.terminate()

    def status(self):
        codes = [c.poll() for c in self.containers]
        if any(c is not None and c != 0 for c in codes):
            return "FAILED"
        if all(c == 0 for c in codes):
            return "COMPLETED"
        return "RUNNING"

    def failed(self):
        return [(i, c) for i, c in enumerate(self.containers) if c.poll() not in (None, 0)]


class CollectiveController:
    def __init__(self, args):
        self.args = args
        self.pod = Pod()
        self.store = None
        self.restarts = 0

    # ------------------------------------------------------------------ topology
    def _local_devices(self):
        a = self.args
        if a.devices:
            devs = []
            for part in str(a.devices).split(","):
                if "-" in part:
                    lo, hi = part.split("-")
                    devs += [str(i) for i in range(int(lo), int(hi) + 1)]
                else:
                    devs.append(part)
            return devs
        if a.nproc_per_node:
            return [str(i) for i in range(a.nproc_per_node)]
        try:
            import torch
            n = torch.cuda.device_count()
        except Exception:  # noqa: BLE001
            n = 0
        return [str(i) for i in range(max(n, 1))]

    def _sync_peers(self, nnodes, my_eps):
        """Returns (node_rank, all endpoints ordered by node rank)."""
        a = self.args
        if nnodes == 1:
            return 0, my_eps
        from ..store import TCPStore
        host, port = a.master.rsplit(":", 1)
        is_master = a.rank == 0 or (a.rank < 0 and a.host == host)
        self.store = TCPStore(host, int(port), is_master=is_master, world_size=nnodes, timeout=a.elastic_timeout * 10)
        gen = f"{a.job_id}/{self.restarts}"
        rank = a.rank if a.rank >= 0 else self.store.add(f"{gen}/next_rank", 1) - 1
        self.store.set(f"{gen}/eps/{rank}", ",".join(my_eps))
        eps = []
        for r in range(nnodes):
            eps += self.store.get(f"{gen}/eps/{r}").decode().split(",")
        return rank, eps

    def build_pod(self):
        a = self.args
        devices = self._local_devices()
        nproc = a.nproc_per_node or len(devices)
        nnodes = int(str(a.nnodes).split(":")[0])
        ports = _free_ports(nproc)
        my_eps = [f"{a.host}:{p}" for p in ports]
        node_rank, eps = self._sync_peers(nnodes, my_eps)
        world = nnodes * nproc
        master = eps[0]      # the trainers' own store is served by global rank 0 on its endpoint
        self.pod = Pod()
        for i in range(nproc):
            rank = node_rank * nproc + i
            env = dict(os.environ)
            env.update({
                "PADDLE_MASTER": master, "PADDLE_GLOBAL_SIZE": str(world), "PADDLE_LOCAL_SIZE": str(nproc),
                "PADDLE_GLOBAL_RANK": str(rank), "PADDLE_LOCAL_RANK": str(i), "PADDLE_NNODES": str(nnodes),
                "PADDLE_CURRENT_ENDPOINT": my_eps[i], "PADDLE_TRAINER_ID": str(rank), "PADDLE_TRAINERS_NUM": str(world),
                "PADDLE_RANK_IN_NODE": str(i), "PADDLE_TRAINER_ENDPOINTS": ",".join(eps),
                "FLAGS_selected_gpus": devices[i % len(devices)], "PADDLE_JOB_ID": a.job_id,
                "PADDLE_RESTART_COUNT": str(self.restarts),
            })
            if a.backend:
                env["PADDLE_DISTRI_BACKEND"] = a.backend
            entry = [sys.executable, "-u", a.training_script, *a.training_script_args]
            self.pod.containers.append(Container(entry, env, os.path.join(a.log_dir, f"workerlog.{rank}")))

    # ------------------------------------------------------------------ run / watch
    def watch(self):
        """Poll the pod; returns its final status."""
        while True:
            st = self.pod.status()
            if st != "RUNNING":
                return st
            time.sleep(self.args.poll_interval)

    def run(self):
        from .watcher import Watcher
        watcher = Watcher(self.args.log_dir, interval=getattr(self.args, "gpu_watch_interval", 30.0)).start()
        try:
            return self._run()
        finally:
            watcher.stop()

    def _run(self):
        a = self.args
        while True:
            self.build_pod()
            self.pod.deploy()
            status = self.watch()
            if status == "COMPLETED":
                self.pod.stop()
                return 0
            failed = self.pod.failed()
            for i, c in failed:
                sys.stderr.write(f"[launch] rank container {i} exited with {c.poll()}; log tail:\n{c.tail()}\n")
            self.pod.stop()
            code = failed[0][1].poll() if failed else 1
            # fault-tolerant / elastic levels rebuild the pod; level <= 0 fails the job (controller.py:119-147)
            if (a.elastic_level > 0 or code == ELASTIC_EXIT_CODE) and self.restarts < a.max_restart:
                self.restarts += 1
                sys.stderr.write(f"[launch] restarting the pod ({self.restarts}/{a.max_restart})\n")
                continue
            return code or 1


def launch(argv=None):
    args = parse_args(argv)
    if args.auto_tuner_json:
        from .auto_tune import run_auto_tuner
        code = run_auto_tuner(args)
        if code:
            sys.exit(code)
        return
    ctl = CollectiveController(args)

    def on_signal(signum, frame):
        ctl.pod.stop()
        sys.exit(128 + signum)
    signal.signal(signal.SIGTERM, on_signal)
    signal.signal(signal.SIGINT, on_signal)
    code = ctl.run()
    if code:
        sys.exit(code)
