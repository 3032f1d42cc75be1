"""Spawn N rank processes on this host (the reference's substitute for a cluster:
test/legacy_test/test_parallel_dygraph_dataparallel.py:100 ``start_local_trainers``), wait with a
timeout, and collect what each rank pickled."""
import os
import pickle
import socket
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def free_port_block(n):
    """First port of ``n`` consecutive ports that are all free right now."""
    for _ in range(50):
        p = free_port()
        ok = True
        for i in range(1, n):
            with socket.socket() as s:
                try:
                    s.bind(("127.0.0.1", p + i))
                except OSError:
                    ok = False
                    break
        if ok:
            return p
    return free_port()


def run_workers(script, nranks, backend="gloo", extra_env=None, timeout=240, args=(), gpus=False, _retry=True):
    try:
        return _run_workers(script, nranks, backend, extra_env, timeout, args, gpus)
    except AssertionError as e:
        # another process can grab a rendezvous port between the probe and the workers' bind
        # (or a loaded machine resets a connection while the ranks build gloo's full mesh): try once more
        transient = ("ddress already in use", "EADDRINUSE", "Connection refused", "Connection reset", "connectFullMesh",
                     "Broken pipe")
        if _retry and any(t in str(e) for t in transient):
            return _run_workers(script, nranks, backend, extra_env, timeout, args, gpus)
        raise


def _run_workers(script, nranks, backend, extra_env, timeout, args, gpus):
    port = free_port_block(nranks)
    eps = ",".join(f"127.0.0.1:{port + i}" for i in range(nranks))
    out = os.path.join(tempfile.mkdtemp(prefix="pdtest_"), "out")
    procs = []
    for r in range(nranks):
        env = dict(os.environ)
        env.update({"PADDLE_TRAINER_ID": str(r), "PADDLE_TRAINERS_NUM": str(nranks), "PADDLE_TRAINER_ENDPOINTS": eps,
                    "PADDLE_CURRENT_ENDPOINT": f"127.0.0.1:{port + r}", "PADDLE_MASTER": f"127.0.0.1:{port}",
                    "PADDLE_DISTRI_BACKEND": backend, "PD_TEST_OUT": out, "PYTHONPATH": ROOT,
                    "FLAGS_selected_gpus": str(r if gpus else 0), "OMP_NUM_THREADS": "2"})
        if not gpus:
            env["CUDA_VISIBLE_DEVICES"] = ""
        env.pop("RANK", None), env.pop("WORLD_SIZE", None)
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "dist_workers", script), *args],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    logs, rcs = [], []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
            o += "\n[timeout]"
        logs.append(o)
        rcs.append(p.returncode)
    if any(rc != 0 for rc in rcs):
        raise AssertionError("worker failed:\n" + "\n-----\n".join(l[-3000:] for l in logs))
    res = []
    for r in range(nranks):
        with open(f"{out}.{r}", "rb") as f:
            res.append(pickle.load(f))
    return res
