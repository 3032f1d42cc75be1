"""Native host runtime: TCP store commands, bucket assignment, watchdog verdicts, reshard planner."""
import ctypes
import threading
import time

import pytest


def test_tcp_store_commands():
    from paddle_b200.distributed.store import StoreTimeoutError, TCPStore
    master = TCPStore("127.0.0.1", 0, is_master=True, world_size=2, timeout=5)
    client = TCPStore("127.0.0.1", master.port, is_master=False, world_size=2, timeout=5)
    client.set("k", b"hello")
    assert master.get("k") == b"hello"
    assert master.add("cnt", 3) == 3 and client.add("cnt", 4) == 7
    assert client.check("k") and not client.check("nope")
    got = {}
    t = threading.Thread(target=lambda: got.setdefault("v", client.get("late")))
    t.start()
    time.sleep(0.2)
    master.set("late", b"x" * 100000)
    t.join(5)
    assert got["v"] == b"x" * 100000
    assert master.delete_key("k") and not master.check("k")
    th = threading.Thread(target=lambda: client.barrier("b0", 2, 5))
    th.start()
    master.barrier("b0", 2, 5)
    th.join(5)
    assert not th.is_alive()
    short = TCPStore("127.0.0.1", master.port, timeout=0.3)
    with pytest.raises(StoreTimeoutError):
        short.get("never-set")
    client.close(), master.close()


def test_assign_group_by_size_native_matches_python():
    import torch
    from paddle_b200.distributed import reducer
    params = [torch.zeros(n, dtype=dt) for n, dt in [(1000, torch.float32), (300000, torch.float32),
                                                       (50, torch.bfloat16), (700000, torch.float32),
                                                       (90000, torch.bfloat16), (10, torch.float32)]]
    groups = reducer.assign_group_by_size(params, [1 << 20, 2 << 20])
    flat = sorted(i for g in groups for i in g)
    assert flat == list(range(len(params)))
    for g in groups:
        assert len({params[i].dtype for i in g}) == 1
    assert groups[0][0] == len(params) - 1          # walk starts from the last parameter


def test_watchdog_reports_hung_collective():
    from paddle_b200.distributed import watchdog
    watchdog.start(timeout_s=0.2, poll_ms=20)
    try:
        ok = watchdog.task_create(0, "all_reduce", 1024)
        watchdog.task_started(ok), watchdog.task_finished(ok)
        hung = watchdog.task_create(0, "all_gather", 4096)
        watchdog.task_started(hung)
        never = watchdog.task_create(1, "broadcast", 16)
        time.sleep(0.6)
        reports = []
        while True:
            r = watchdog.poll()
            if r is None:
                break
            reports.append(r)
        assert any("started-but-not-finished" in r and "all_gather" in r and "last_done=all_reduce" in r for r in reports)
        assert any("timeout-not-started" in r and "broadcast" in r for r in reports)
        with pytest.raises(watchdog.CommTimeoutError):
            h2 = watchdog.task_create(2, "reduce", 8)
            time.sleep(0.5)
            watchdog.check()
    finally:
        watchdog.stop()


def test_reshard_planner():
    from paddle_b200.ops import _lib
    rt = _lib.runtime()
    out = (ctypes.c_int * 30)()

    def plan(src, dst):
        n = rt.pd_plan_reshard((ctypes.c_int * len(src))(*src), (ctypes.c_int * len(dst))(*dst), len(src), out, 10)
        return [(out[3 * i], out[3 * i + 1], out[3 * i + 2]) for i in range(n)]
    assert plan([0], [-1]) == [(1, 0, 0)]                 # s -> r : all_gather
    assert plan([-2], [-1]) == [(2, 0, -1)]               # p -> r : all_reduce
    assert plan([-2], [1]) == [(3, 0, 1)]                 # p -> s : reduce_scatter
    assert plan([-1], [0]) == [(4, 0, 0)]                 # r -> s : slice
    assert plan([0], [1]) == [(5, 0, 1)]                  # s -> s : all_to_all
    assert plan([0, -2], [-1, -1]) == [(2, 1, -1), (1, 0, 0)]
    assert rt.pd_comm_static_check(1, 8, 16, 0, 2, 0) == 0 and rt.pd_comm_static_check(1, 8, 8, 0, 2, 0) == 3


def test_push_cta_count_rule(monkeypatch):
    """Number of communication CTAs of the all-gather GEMM: a per-degree base, plus SMs the GEMM's last wave leaves
    idle, never more than there are push jobs, none for a launch that does not push; the environment overrides.
    The multicast push issues one store per 16 bytes whatever the degree and keeps its small base."""
    from paddle_b200.parallel import fused_linear_impl as FL
    monkeypatch.setattr(FL, "_sms", lambda: 148)
    monkeypatch.delenv("PD_AG_COMM_CTAS", raising=False)
    assert FL._comm_ctas(8, 96, 28, True) == 28            # qkv at TP8: one wave of 96 tiles, 52 SMs idle, 28 jobs
    assert FL._comm_ctas(8, 352, 28, True) == 28           # gate_up at TP8: 3 waves of <= 118
    assert FL._comm_ctas(4, 192, 24, True) == 24
    assert FL._comm_ctas(2, 768, 16, True) == 8            # two ranks keep the measured setting
    assert FL._comm_ctas(8, 96, 28, False) == 0
    c = FL._comm_ctas(8, 5000, 28, True)                   # a large GEMM: base plus what keeps the wave count (41)
    assert c == 26 and -(-5000 // (148 - c)) == -(-5000 // (148 - 24))
    for mode, table in ((0, FL._COMM_BASE), (1, FL._COMM_VEC), (2, FL._COMM_MC)):
        for n, tiles, jobs in [(8, 96, 28), (8, 352, 32), (4, 704, 24), (2, 768, 128), (8, 1, 4)]:
            c = FL._comm_ctas(n, tiles, jobs, True, mode)
            assert 1 <= c <= max(jobs, 1) or c == table[n]
            assert 148 - c >= 1
    assert FL._comm_ctas(8, 192, 32, True, 2) == FL._COMM_MC[8]      # multicast: no growth with the degree
    assert FL._comm_ctas(8, 96, 32, True, 1) == 32                   # vector push takes the idle SMs, up to the jobs
    monkeypatch.setenv("PD_AG_COMM_CTAS", "8")
    monkeypatch.setattr(FL, "N_COMM", 8)
    assert FL._comm_ctas(8, 96, 28, True) == 8


@pytest.mark.parametrize("sanitizer", ["address", "thread"])
def test_runtime_under_sanitizer(sanitizer):
    """The C++ host runtime (TCP store with its server / waiter threads, watchdog, bucket assignment, reshard
    planner) rebuilt with AddressSanitizer / ThreadSanitizer passes the same tests with no report."""
    import os
    import subprocess
    import sys

    from paddle_b200.ops import build
    lib = build.sanitizer_runtime_library(sanitizer)
    if not lib:
        pytest.skip(f"no compiler with the {sanitizer} sanitizer run-time is installed")
    build.build_runtime(sanitize=sanitizer)
    env = dict(os.environ, PD_RUNTIME_SANITIZER=sanitizer, LD_PRELOAD=lib, CUDA_VISIBLE_DEVICES="",
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=23",
               TSAN_OPTIONS="exitcode=23:report_signal_unsafe=0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider",
                        os.path.join(root, "tests", "test_runtime_cpu.py"), "-k",
                        "tcp_store or assign_group or watchdog or reshard_planner"],
                       env=env, cwd=root, capture_output=True, text=True, timeout=600)
    report = [l for l in (p.stdout + p.stderr).splitlines() if "Sanitizer" in l and ("ERROR" in l or "WARNING" in l)]
    assert p.returncode == 0 and not report, (p.stdout[-1500:], p.stderr[-1500:])
