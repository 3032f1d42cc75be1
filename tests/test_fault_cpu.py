"""Failure detection and recovery, with every failure made on the host (a rank that exits or never joins, a
membership change in a fake key-value service): launcher restart + resume from checkpoint, bounded-time error on
a missing peer, elastic manager state machine, spawn error propagation."""
import os
import subprocess
import sys
import tempfile
import time
import types

import numpy as np
import pytest

from dist_utils import ROOT, run_workers


def _launch(out, mode, extra=()):
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", PADDLE_DISTRI_BACKEND="gloo", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "paddle_b200.distributed.launch", "--nproc_per_node", "2", "--log_dir",
           os.path.join(out, "log"), *extra, os.path.join(ROOT, "tests", "dist_workers", "elastic_train.py"), out, mode]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)


def _losses(out):
    return [float(l.split()[1]) for l in open(os.path.join(out, "loss.txt"))], \
        [int(l.split()[0]) for l in open(os.path.join(out, "loss.txt"))]


def test_launcher_restart_resumes_from_checkpoint():
    ref = tempfile.mkdtemp()
    r = _launch(ref, "clean")
    assert r.returncode == 0, r.stderr[-2000:]
    out = tempfile.mkdtemp()
    r = _launch(out, "crash", ("--elastic_level", "1", "--max_restart", "2"))
    assert r.returncode == 0, r.stderr[-2000:]
    assert "restarting the pod (1/2)" in r.stderr
    (l_ref, s_ref), (l_out, s_out) = _losses(ref), _losses(out)
    assert s_ref == s_out == list(range(6))
    assert np.allclose(l_ref, l_out, atol=1e-6), (l_ref, l_out)
    assert sorted(os.listdir(os.path.join(out, "log"))) == ["workerlog.0", "workerlog.1"]


def test_launcher_fails_without_elastic_level():
    out = tempfile.mkdtemp()
    r = _launch(out, "crash")
    assert r.returncode != 0 and "restarting" not in r.stderr
    assert "exited with 3" in r.stderr


def test_missing_peer_ends_collective_in_bounded_time():
    res = run_workers("peer_missing.py", 2, timeout=120)
    assert res[1] == {"left": True}
    assert res[0]["first"] == [2.0] * 4
    assert res[0]["error"] is not None and res[0]["elapsed"] < 30, res[0]


def _args(**kw):
    base = dict(np="2", job_id="t", host="10.0.0.1", elastic_timeout=1, elastic_level=None, elastic_server="fake")
    base.update(kw)
    return types.SimpleNamespace(**base)


class _FakeLauncher:
    def __init__(self):
        self.code, self.stopped, self.launched = None, 0, 0

    def launch(self):
        self.launched += 1

    def watch(self):
        return self.code

    def stop(self):
        self.stopped += 1


def test_elastic_manager_fault_tolerance_and_scaling():
    from paddle_b200.distributed.fleet.elastic.manager import ElasticManager, ElasticStatus, MemoryKV
    kv = MemoryKV()
    a = ElasticManager(_args(host="10.0.0.1"), kv)
    b = ElasticManager(_args(host="10.0.0.2"), kv)
    assert a.wait() and b.wait()
    assert a.np == 2 and os.environ["PADDLE_TRAINERS_NUM"] == "2"
    la = _FakeLauncher()
    a.run(la)
    assert la.launched == 1
    b.exit()                                   # the peer leaves: below np -> HOLD (fault tolerance)
    assert a.watch() == ElasticStatus.HOLD and la.stopped >= 1
    assert not a.wait()                        # nobody comes back within elastic_timeout
    c = ElasticManager(_args(host="10.0.0.3"), kv)
    assert a.wait() and sorted(a.trainers.split(",")) == ["10.0.0.1:6170", "10.0.0.3:6170"]
    la.code = 0
    assert a.watch() == ElasticStatus.COMPLETED
    a.exit(completed=True), c.exit()
    # elastic range 1:2 -> losing one host restarts with the survivors instead of holding
    kv2 = MemoryKV()
    d = ElasticManager(_args(np="1:2", host="10.0.1.1"), kv2)
    e = ElasticManager(_args(np="1:2", host="10.0.1.2"), kv2)
    assert d.wait() and d.np == 2
    ld = _FakeLauncher()
    d.run(ld)
    e.exit()
    assert d.watch() == ElasticStatus.RESTART
    assert d.wait() and d.np == 1 and d.trainers == "10.0.1.1:6170"
    ld.code = 101
    assert d.watch() == ElasticStatus.RESTART    # trainers asked for a relaunch through the elastic exit code
    d.exit()


def test_elastic_lease_expires_without_heartbeat():
    from paddle_b200.distributed.fleet.elastic.manager import MemoryKV
    kv = MemoryKV()
    lease = kv.lease(0.2)
    kv.put("/paddle/j/nodes/x", "h:1", lease=lease)
    events = []
    kv.add_watch_prefix_callback("/paddle/j/nodes", events.append)
    assert len(kv.get_prefix("/paddle/j/nodes")) == 1
    time.sleep(0.3)
    assert kv.get_prefix("/paddle/j/nodes") == [] and events and events[0]["type"] == "delete"


def _spawn_ok(path):
    import paddle_b200.distributed as dist
    import torch
    dist.init_parallel_env()
    t = torch.tensor([float(dist.get_rank() + 1)])
    dist.all_reduce(t)
    with open(f"{path}.{dist.get_rank()}", "w") as f:
        f.write(str(float(t)))


def _spawn_bad(path):
    raise ValueError("boom from the child")


def test_spawn_runs_and_propagates_errors():
    import paddle_b200.distributed as dist
    base = os.path.join(tempfile.mkdtemp(), "o")
    env = {"CUDA_VISIBLE_DEVICES": "", "PADDLE_DISTRI_BACKEND": "gloo"}
    dist.spawn(_spawn_ok, args=(base,), nprocs=2, env=env)
    assert [open(f"{base}.{r}").read() for r in range(2)] == ["3.0", "3.0"]
    with pytest.raises(RuntimeError, match="boom from the child"):
        dist.spawn(_spawn_bad, args=(base,), nprocs=2, env=env)


def test_pipeline_schedules_are_deadlock_free_and_have_the_expected_bubble():
    """Host-side check of the generated per-rank orders: every step's input is produced earlier somewhere, the
    greedy makespan is 2*M*V + 2*(P-1) virtual steps (the interleaved bubble), and a broken order is reported."""
    from paddle_b200.distributed.fleet.meta_parallel import pipeline_schedules as S
    unit = {"F": 1, "B": 1, "Bx": 1, "W": 1}
    for P, V, M in [(2, 2, 4), (4, 2, 8), (4, 3, 8), (8, 2, 16)]:
        assert S.validate(S.interleaved_1f1b, P, V, M, cost=unit) == 2 * M * V + 2 * (P - 1)
        steps = S.interleaved_1f1b(P, V, M, 0)
        warm = next(i for i, s in enumerate(steps) if s[0] == "B")
        assert warm == min((P - 1) * 2 + (V - 1) * P, M * V) + 1          # warm-up forwards + the first steady forward
        assert sorted(s for s in steps if s[0] == "F") == sorted(("F", c, m) for c in range(V) for m in range(M))
    for P, M in [(2, 4), (4, 8)]:
        assert S.validate(S.one_f_one_b, P, 1, M, cost=unit) == 2 * M + 2 * (P - 1)
    # with a backward that costs two forwards, 1F1B idles 3 * (P - 1) units; ZB-H1 fills part of that with the
    # postponed weight gradients, and every Bx is matched by exactly one later W on the same rank
    for P, M in [(2, 2), (4, 4), (4, 8), (8, 16)]:
        assert S.validate(S.one_f_one_b, P, 1, M) == 3 * M + 3 * (P - 1)
        zb = S.validate(S.zero_bubble_h1, P, 1, M)
        assert 3 * M + (P - 1) <= zb < 3 * M + 3 * (P - 1)
        for r in range(P):
            steps = S.zero_bubble_h1(P, 1, M, r)
            assert sorted(m for k, _, m in steps if k == "Bx") == sorted(m for k, _, m in steps if k == "W")
            assert sorted(m for k, _, m in steps if k in ("B", "Bx")) == list(range(M))

    def lost_w(P, V, M, rank):
        return [("F", 0, 0), ("Bx", 0, 0)]
    import pytest
    with pytest.raises(RuntimeError, match="no W step"):
        S.validate(lost_w, 1, 1, 1)

    def broken(P, V, M, rank):           # backward before its forward
        return [("B", 0, 0), ("F", 0, 0)]
    import pytest
    with pytest.raises(RuntimeError, match="before its forward"):
        S.validate(broken, 2, 1, 1)

    def cyclic(P, V, M, rank):           # stage 1 wants the gradient path first, stage 0 never produces for it
        return [("F", 0, 0), ("B", 0, 0)] if rank == 0 else [("F", 0, 1), ("F", 0, 0), ("B", 0, 0)]
    with pytest.raises(RuntimeError, match="deadlocks"):
        S.validate(cyclic, 2, 1, 2)
    with pytest.raises(ValueError):
        S.interleaved_1f1b(4, 2, 6, 0)


def test_launcher_gpu_watcher_writes_samples(tmp_path):
    import time

    from paddle_b200.distributed.launch.watcher import Watcher
    fake = lambda: [{"index": "0", "utilization.gpu": "97", "memory.used": "1000"},       # noqa: E731
                    {"index": "1", "utilization.gpu": "3", "memory.used": "10"}]
    w = Watcher(str(tmp_path), interval=0.05, sampler=fake, devices=[0]).start()
    time.sleep(0.3)
    w.stop()
    lines = (tmp_path / "gpu.log").read_text().strip().splitlines()
    assert w.samples >= 2 and len(lines) == w.samples and all("index=0 utilization.gpu=97" in l for l in lines)
    silent = Watcher(str(tmp_path / "none"), interval=0.05, sampler=lambda: []).start()
    time.sleep(0.15)
    silent.stop()
    assert not (tmp_path / "none" / "gpu.log").exists()


def test_corrupt_checkpoint_shard_is_reported_by_name(tmp_path):
    """Host-injected failure: a bit flip and a truncation in a distributed-checkpoint shard are detected at load."""
    import numpy as np
    import pytest

    import paddle_b200 as paddle
    from paddle_b200.distributed import checkpoint as ckpt
    sd = {"w": paddle.to_tensor(np.arange(4096, dtype="float32")), "step": 7}
    ckpt.save_state_dict(sd, str(tmp_path))
    shard = next(p for p in tmp_path.iterdir() if p.name.endswith(".distcp"))
    assert (tmp_path / (shard.name + ".crc")).exists()
    fresh = {"w": paddle.zeros([4096]), "step": 0}
    ckpt.load_state_dict(fresh, str(tmp_path))
    assert fresh["step"] == 7 and float(fresh["w"][100]) == 100.0
    raw = bytearray(shard.read_bytes())
    raw[len(raw) // 2] ^= 0x40
    shard.write_bytes(bytes(raw))
    with pytest.raises(ckpt.CheckpointCorruptError, match=shard.name):
        ckpt.load_state_dict({"w": paddle.zeros([4096]), "step": 0}, str(tmp_path))
    shard.write_bytes(bytes(raw[:100]))
    with pytest.raises(ckpt.CheckpointCorruptError, match="corrupt"):
        ckpt.load_state_dict({"w": paddle.zeros([4096]), "step": 0}, str(tmp_path))
    (tmp_path / (shard.name + ".crc")).unlink()                 # without the side file the decoder still reports it
    with pytest.raises(ckpt.CheckpointCorruptError, match="cannot be decoded"):
        ckpt.load_state_dict({"w": paddle.zeros([4096]), "step": 0}, str(tmp_path))


def test_checkpoint_load_picks_newest_of_eleven_versions(tmp_path, monkeypatch):
    """Eleven periodic saves into one directory (ids 0..10): loading without an id restores version 10 - ids compare as
    numbers, '9' does not beat '10' - and reads no other version's files; an explicit id still selects an old one."""
    import numpy as np

    import paddle_b200 as paddle
    from paddle_b200.distributed import checkpoint as ckpt
    import importlib
    L = importlib.import_module("paddle_b200.distributed.checkpoint.load_state_dict")
    for v in range(11):
        ckpt.save_state_dict({"w": paddle.to_tensor(np.full(8, float(v), dtype="float32")), "step": v}, str(tmp_path))
    assert sorted(int(p.name.split(".")[0]) for p in tmp_path.iterdir() if p.name.endswith(".metadata")) == list(range(11))
    assert L.get_max_id(str(tmp_path)) == 10
    read = []
    real = L._load_verified
    monkeypatch.setattr(L, "_load_verified", lambda fn: (read.append(fn.rsplit("/", 1)[1]), real(fn))[1])
    fresh = {"w": paddle.zeros([8]), "step": -1}
    ckpt.load_state_dict(fresh, str(tmp_path))
    assert fresh["step"] == 10 and float(fresh["w"][3]) == 10.0
    assert sorted(set(read)) == ["0_10.distcp", "10.metadata"], read
    merged = ckpt.load_merged_state_dict(str(tmp_path))
    assert float(merged["w"][0]) == 10.0
    old = {"w": paddle.zeros([8]), "step": -1}
    ckpt.load_state_dict(old, str(tmp_path), unique_id=9)
    assert old["step"] == 9 and float(old["w"][0]) == 9.0


def test_weight_grad_store_defers_and_matches_plain_backward():
    """Split backward of linear layers: with the store enabled, backward yields only input gradients; running the
    queued closures afterwards gives the same weight / bias gradients as an ordinary backward."""
    import torch
    import paddle_b200 as paddle
    from paddle_b200.ops.functional import WeightGradStore
    paddle.seed(3)
    net = paddle.nn.Sequential(paddle.nn.Linear(6, 5), paddle.nn.Tanh(), paddle.nn.Linear(5, 4))
    x = paddle.randn([3, 6])
    x.stop_gradient = False
    net(x).square().sum().backward()
    ref = [p.grad.clone() for p in net.parameters()] + [x.grad.clone()]
    for p in net.parameters():
        p.clear_gradient()
    x.clear_gradient()
    WeightGradStore.split = WeightGradStore.enabled = True
    try:
        net(x).square().sum().backward()
        assert all(p.grad is None or not bool(p.grad.any()) for p in net.parameters())
        assert torch.allclose(x.grad, ref[-1], atol=1e-6)
        batch = WeightGradStore.pop()
        assert len(batch) == 2
    finally:
        WeightGradStore.split = WeightGradStore.enabled = False
    WeightGradStore.run(batch)
    for p, g in zip(net.parameters(), ref):
        assert torch.allclose(p.grad, g, atol=1e-6)


def test_native_process_group_task_timeout_error_and_abort(tmp_path):
    """The native process group against stand-in NCCL / CUDA-runtime libraries (host-injected failures, no GPU): a
    collective completes and its task is forgotten; a stalled one times out within the bound, the failure is published
    for the peers and the communicator is aborted; an asynchronous communicator error is reported as such; a failing
    NCCL call surfaces its result code; an aborted group refuses further calls."""
    import ctypes
    import os
    import subprocess
    import time

    import pytest
    import torch

    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fakes")
    libs = {}
    for name in ("fake_nccl", "fake_cudart"):
        out = str(tmp_path / f"lib{name}.so")
        subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", out, os.path.join(here, name + ".c")], check=True)
        libs[name] = out
    from paddle_b200.distributed import native_pg as N
    N.load(libs["fake_nccl"], libs["fake_cudart"])
    fn, fc = ctypes.CDLL(libs["fake_nccl"]), ctypes.CDLL(libs["fake_cudart"])

    class Store(dict):
        def set(self, k, v): self[k] = v
        def get(self, k): return self[k]
        def check(self, keys): return all(k in self for k in keys)

    store = Store()
    pg = N.NativeProcessGroup(0, 1, device=0, store=store, name="g0")
    assert "pd/nccl_id/g0" in store and len(store["pd/nccl_id/g0"]) == 128
    x = torch.arange(8, dtype=torch.float32)
    out = torch.zeros(8)
    pg.all_gather(out, x)                                  # sync_op: issued on the comm stream, waited for
    assert torch.equal(out, x) and pg.inflight() == 0
    t = pg.all_reduce(x, sync_op=False)
    assert t.is_completed() and t.wait(timeout=1.0) and pg.inflight() == 0
    pg.broadcast(x, 0, use_calc_stream=True)
    # a failing NCCL call is reported with its result code
    fn.fake_nccl_set(0, 3)
    with pytest.raises(N.CommError, match="nccl result 3"):
        pg.all_reduce(x)
    # asynchronous communicator error while waiting
    fc.fake_cuda_stall(1)
    t = pg.all_reduce(x, sync_op=False)
    assert not t.is_completed()
    fn.fake_nccl_set(1, 0)
    with pytest.raises(N.CommError) as e:
        t.wait(timeout=5.0)
    assert e.value.kind == "comm_error" and pg.aborted and fn.fake_nccl_aborts() == 1
    assert b"comm_error" in store["pd/comm_error/g0"]
    with pytest.raises(N.CommError, match="aborted"):
        pg.all_reduce(x)
    pg.destroy()
    # timeout: bounded, then abort; a second group learns about it from the store before its next call
    fn.fake_nccl_set(0, 0)
    store2 = Store()
    pg2 = N.NativeProcessGroup(0, 1, store=store2, name="g1")
    t = pg2.reduce_scatter(out, x, sync_op=False)
    t0 = time.perf_counter()
    with pytest.raises(N.CommError) as e:
        t.wait(timeout=0.2)
    assert e.value.kind == "timeout" and 0.15 < time.perf_counter() - t0 < 2.0 and fn.fake_nccl_aborts() == 2
    fc.fake_cuda_stall(0)
    peer = N.NativeProcessGroup(0, 1, store=store2, name="g1", unique_id=store2["pd/nccl_id/g1"])
    with pytest.raises(N.CommError, match="a peer reported"):
        peer.all_reduce(x)
    assert peer.aborted
    peer.destroy(), pg2.destroy()


def test_zero_bubble_v_schedule_properties():
    """The zero-bubble V schedule: valid for every (P, M) tried (no deadlock, every Bx has its W), every rank runs
    each of its 2 M forwards / input-gradient halves / weight-gradient halves exactly once, its makespan stays within
    P + 3 units of the bubble-free 6 M and below interleaved 1F1B with the same two chunks, and the placement is the V."""
    from paddle_b200.distributed.fleet.meta_parallel import pipeline_schedules as S
    place = S.Placement(4, 2, "zigzag")
    assert [place.vs(0, r) for r in range(4)] == [0, 1, 2, 3] and [place.vs(1, r) for r in range(4)] == [7, 6, 5, 4]
    assert all(place.owner(place.vs(c, r)) == (r, c) for c in range(2) for r in range(4))
    for P, M in ((2, 2), (2, 4), (3, 6), (4, 4), (4, 8), (8, 8), (8, 16)):
        span = S.validate(S.zero_bubble_v, P, 2, M)
        assert span <= 6 * M + P + 3, (P, M, span)
        assert span < S.validate(S.interleaved_1f1b, P, 2, M) if M % P == 0 else True
        for r in range(P):
            steps = S.zero_bubble_v(P, 2, M, r)
            for kind in ("F", "Bx", "W"):
                got = sorted((c, m) for k, c, m in steps if k == kind)
                assert got == sorted((c, m) for c in range(2) for m in range(M)), (P, M, r, kind)
            # memory: bounded independently of M - at most 3 P chunk activations alive on a rank (first-chunk forwards
            # stop at 2 P, second-chunk forwards are never held back)
            alive = peak = 0
            for k, _, _ in steps:
                alive += 1 if k == "F" else (-1 if k == "W" else 0)
                peak = max(peak, alive)
            assert peak <= 3 * P, (P, M, r, peak)
    with pytest.raises(ValueError):
        S.zero_bubble_v(4, 3, 8, 0)
