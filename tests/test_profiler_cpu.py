"""Profiler: range algebra, statistics over hand-written timelines (model phases, operator / kernel tables,
communication-computation overlap), chrome-trace round trip, a real CPU recording, the benchmark timer and its data
loader hooks (reference behaviour: python/paddle/profiler/, test/legacy_test/test_profiler_statistic.py,
test_newprofiler.py)."""
import json
import time

import numpy as np
import pytest

import paddle_b200 as paddle
from paddle_b200 import profiler
from paddle_b200.profiler import statistic_helper as sh
from paddle_b200.profiler.profiler_statistic import (DeviceEvent, HostEvent, MemEvent, StatisticData, TracerEventType as T, _build_table,
                                                     build_tree, events_from_chrome_trace)


def test_range_algebra():
    assert sh.merge_self_ranges([(5, 7), (1, 3), (2, 4), (7, 9), (20, 20)]) == [(1, 4), (5, 9)]
    assert sh.sum_ranges([(1, 4), (5, 9)]) == 7
    assert sh.merge_ranges([(1, 3)], [(2, 6), (8, 9)]) == [(1, 6), (8, 9)]
    assert sh.intersection_ranges([(0, 10), (20, 30)], [(5, 25), (28, 40)]) == [(5, 10), (20, 25), (28, 30)]
    assert sh.subtract_ranges([(0, 10), (20, 30)], [(2, 4), (8, 22), (29, 35)]) == [(0, 2), (4, 8), (22, 29)]
    assert sh.subtract_ranges([(0, 10)], []) == [(0, 10)] and sh.intersection_ranges([], [(0, 1)]) == []
    rng = np.random.default_rng(0)
    for _ in range(20):                                  # against a bitmap
        a = [(int(s), int(s + d)) for s, d in zip(rng.integers(0, 90, 6), rng.integers(0, 12, 6))]
        b = [(int(s), int(s + d)) for s, d in zip(rng.integers(0, 90, 6), rng.integers(0, 12, 6))]
        bm = lambda rs: np.array([any(s <= t < e for s, e in rs) for t in range(110)])
        assert sh.sum_ranges(sh.intersection_ranges(a, b)) == int((bm(a) & bm(b)).sum())
        assert sh.sum_ranges(sh.subtract_ranges(a, b)) == int((bm(a) & ~bm(b)).sum())
        assert sh.sum_ranges(sh.merge_ranges(a, b)) == int((bm(a) | bm(b)).sum())


def _timeline():
    """One step: data loader, forward (two matmuls, an all-gather GEMM overlapping a plain kernel), backward,
    optimizer; times in ns."""
    k = lambda name, s, e, typ=T.Kernel: DeviceEvent(name, typ, s, e)
    ev = [
        HostEvent("ProfileStep#0", T.ProfileStep, 0, 1000),
        HostEvent("Dataloader#next", T.Dataloader, 0, 100),
        HostEvent("Llama.forward", T.Forward, 100, 400),
        HostEvent("pd::matmul", T.Operator, 110, 150, device=[k("gemm2_bf16_kernel", 200, 300)]),
        HostEvent("pd::matmul", T.Operator, 160, 220, device=[k("gemm2_bf16_kernel", 300, 420)]),
        HostEvent("pd::allgather_linear", T.Operator, 230, 300, device=[k("ag_gemm_kernel", 420, 560)]),
        HostEvent("aten::copy_", T.Operator, 310, 330, device=[k("Memcpy DtoD", 430, 450, T.Memcpy)]),
        HostEvent("my_range", T.PythonUserDefined, 340, 390, device=[k("rms_norm_fwd_kernel", 500, 600)]),
        HostEvent("autograd::engine::evaluate_function: MmBackward0", T.Backward, 400, 700,
                  device=[k("gemm2_bf16_kernel", 600, 700), k("ncclDevKernel_AllReduce", 650, 800)]),
        HostEvent("Optimizer.step#AdamW", T.Optimization, 700, 900, device=[k("adamw_multi_kernel", 800, 900)]),
    ]
    return ev


def test_statistics_on_a_hand_written_timeline():
    ev = _timeline()
    roots = build_tree(ev)[0]
    assert [r.name for r in roots] == ["ProfileStep#0"]
    fwd = [c for c in roots[0].children if c.type == T.Forward][0]
    assert [c.name for c in fwd.children] == ["pd::matmul", "pd::matmul", "pd::allgather_linear", "aten::copy_", "my_range"]
    sd = StatisticData(ev, [MemEvent(10, "gpu", 1000), MemEvent(20, "gpu", 500), MemEvent(30, "gpu", -1200), MemEvent(40, "cpu", 64)])
    es = sd.event_summary
    mm = es.items["pd::matmul"]
    assert (mm.call, mm.cpu_time, mm.max_cpu_time, mm.min_cpu_time, mm.gpu_time) == (2, 100, 60, 40, 220)
    assert es.items["pd::matmul"].devices["gemm2_bf16_kernel"].call == 2
    assert es.kernel_items["gemm2_bf16_kernel"].call == 3 and es.kernel_items["gemm2_bf16_kernel"].gpu_time == 320
    assert es.memory_manipulation_items["Memcpy DtoD"].gpu_time == 20
    assert es.userdefined_items["my_range"].cpu_time == 50 and es.userdefined_items["my_range"].gpu_time == 100
    mp = es.model_perspective_items
    assert mp["Forward"].cpu_time == 300 and mp["Forward"].gpu_time == 100 + 120 + 140 + 20 + 100
    assert mp["Backward"].gpu_time == 250 and mp["Optimization"].cpu_time == 200 and mp["Dataloader"].cpu_time == 100
    assert mp["ProfileStep"].cpu_time == 1000 and mp["Others"].cpu_time == 1000 - 900
    ds = sd.distributed_summary
    # communication kernels: ag_gemm 420-560, nccl 650-800 -> 290; computation: 200-420, 500-700, 800-900 -> 520
    assert ds.communication_ns == 290 and ds.computation_ns == 520
    assert ds.overlap_ns == (560 - 500) + (700 - 650) and ds.exposed_ns == 290 - 110
    assert sd.memory_summary.peak_allocated["gpu"] == 1500 and sd.memory_summary.free_calls["gpu"] == 1
    trs = sd.time_range_summary
    assert trs.get_cpu_range_sum(T.Operator) == 40 + 60 + 70 + 20 and trs.get_gpu_range_sum(T.Kernel) == 700 and trs.total_ns == 1000
    table = _build_table(sd, profiler.SortedKeys.GPUTotal, time_unit="ns")
    for title in ("Overview Summary", "Model Summary", "Distribution Summary", "Operator Summary", "Kernel Summary",
                  "Memory Manipulation Summary", "UserDefined Summary", "Memory Summary"):
        assert title in table
    op_part = table[table.index("Operator Summary"):table.index("Kernel Summary")]
    assert op_part.index("pd::matmul") < op_part.index("pd::allgather_linear") < op_part.index("aten::copy_")     # by GPU total
    assert "    gemm2_bf16_kernel" in op_part                                               # operator detail
    only = _build_table(sd, views=[profiler.SummaryView.KernelView], time_unit="us")
    assert "Kernel Summary" in only and "Operator Summary" not in only


def test_chrome_trace_round_trip(tmp_path):
    doc = {"traceEvents": [
        {"ph": "X", "cat": "user_annotation", "name": "ProfileStep#3", "ts": 0, "dur": 100, "tid": 1},
        {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": 10, "dur": 20, "tid": 1},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernel", "ts": 15, "dur": 5, "tid": 1, "args": {"correlation": 7}},
        {"ph": "X", "cat": "kernel", "name": "gemm2_bf16_kernel", "ts": 40, "dur": 30, "tid": 7, "args": {"correlation": 7, "stream": 7}},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaMemcpyAsync", "ts": 60, "dur": 5, "tid": 1, "args": {"correlation": 8}},
        {"ph": "X", "cat": "gpu_memcpy", "name": "Memcpy HtoD", "ts": 75, "dur": 5, "tid": 7, "args": {"correlation": 8}},
        {"ph": "i", "name": "[memory]", "ts": 12, "args": {"Device Type": 1, "Bytes": 4096, "Total Allocated": 4096}},
        {"ph": "s", "cat": "ac2g", "name": "ac2g", "ts": 15, "id": 7},
    ]}
    host, mem = events_from_chrome_trace(doc)
    launch = [h for h in host if h.name == "cudaLaunchKernel"][0]
    assert launch.type == T.CudaRuntime and launch.device[0].name == "gemm2_bf16_kernel" and launch.device[0].duration == 30000
    assert mem[0].place == "gpu" and mem[0].increase_bytes == 4096
    path = tmp_path / "t.json"
    path.write_text(json.dumps(doc))
    res = profiler.load_profiler_result(str(path))
    es = res.statistic_data.event_summary
    assert es.items["aten::mm"].gpu_time == 30000 and es.items["aten::mm"].devices["gemm2_bf16_kernel"].call == 1
    assert "Memcpy HtoD" in es.memory_manipulation_items
    assert "aten::mm" in res.summary(views=profiler.SummaryView.OperatorView)


def test_real_recording_on_cpu(tmp_path):
    lin = paddle.nn.Linear(16, 16)
    opt = paddle.optimizer.AdamW(parameters=lin.parameters(), learning_rate=1e-3)
    ds = paddle.io.TensorDataset([paddle.randn([12, 16]), paddle.randn([12, 16])])
    loader = paddle.io.DataLoader(ds, batch_size=4)
    traces = []
    prof = profiler.Profiler(targets=[profiler.ProfilerTarget.CPU], scheduler=(1, 3),
                             on_trace_ready=lambda p: traces.append(p.summary(views=[profiler.SummaryView.ModelView,
                                                                                      profiler.SummaryView.OperatorView,
                                                                                      profiler.SummaryView.UDFView])))
    with prof:
        for x, y in loader:
            with profiler.RecordEvent("my_forward", profiler.TracerEventType.Forward):
                loss = ((lin(x) - y) ** 2).mean()
            with profiler.RecordEvent("user_block"):
                loss.backward()
            opt.step()
            opt.clear_grad()
            prof.step(num_samples=4)
    assert len(traces) == 1 and prof.step_num == 3
    t = traces[0]
    assert "Model Summary" in t and "Forward" in t and "Optimization" in t and "Dataloader" in t and "user_block" in t
    assert "aten::addmm" in t or "aten::linear" in t or "aten::mm" in t
    assert not profiler.in_profiler_mode()
    out = tmp_path / "trace"
    handler = profiler.export_chrome_tracing(str(out))
    handler(prof)
    files = list(out.iterdir())
    assert len(files) == 1 and files[0].name.endswith(".paddle_trace.json") and "traceEvents" in json.load(open(files[0]))

    @profiler.RecordEvent("decorated")
    def f():
        return 3
    assert f() == 3


def test_benchmark_timer_and_loader_hooks(capsys):
    bench = profiler.benchmark()
    ds = paddle.io.TensorDataset([paddle.randn([64, 4])])

    class Slow(paddle.io.Dataset):
        def __len__(self):
            return 16

        def __getitem__(self, i):
            time.sleep(0.002)
            return np.zeros(2, "float32")
    loader = paddle.io.DataLoader(Slow(), batch_size=2)
    prof = profiler.Profiler(timer_only=True)
    prof.start()
    infos = []
    for i, _ in enumerate(loader):
        time.sleep(0.001)
        prof.step(num_samples=2)
        if i % 4 == 3:
            infos.append(prof.step_info(unit="samples"))
    prof.stop()
    assert len(infos) == 2 and all(s.startswith("reader_cost:") and "samples/s" in s for s in infos)
    reader = float(infos[0].split()[1])
    batch = float(infos[0].split()[4])
    ips = float(infos[0].split()[7])
    assert 0.003 < reader < batch and ips == pytest.approx(2 / batch, rel=0.05)
    ev = profiler.timer.Event()
    ev.skip_iter = 2
    for t in (1.0, 1.0, 0.5, 0.25, 0.25):
        ev.record_reader(t / 10)
        ev.record_batch(t, 8)
    s = ev.get_summary()
    assert s["steps"] == 3 and s["batch_summary"] == dict(avg=pytest.approx(1 / 3), max=0.5, min=0.25)
    assert s["ips_summary"]["avg"] == pytest.approx(24.0) and s["ips_summary"]["max"] == 32.0
    assert "Perf Summary over 3 steps" in profiler.timer.Benchmark.format_summary(s)
    assert bench.current_event is None                       # stop() closed the loop's event


def test_get_profiler_from_config(tmp_path):
    cfg = tmp_path / "p.json"
    cfg.write_text(json.dumps({"targets": ["CPU"], "scheduler": {"closed": 1, "ready": 1, "record": 2, "repeat": 1}, "timer_only": True,
                               "on_trace_ready": {"export_chrome_tracing": {"dir_name": str(tmp_path / "o")}}}))
    p = profiler.get_profiler(str(cfg))
    assert p.timer_only and p.targets == [profiler.ProfilerTarget.CPU]
    assert [p.scheduler(i).name for i in range(5)] == ["CLOSED", "READY", "RECORD", "RECORD_AND_RETURN", "CLOSED"]
    assert isinstance(profiler.get_profiler(str(tmp_path / "missing.json")), profiler.Profiler)
    assert profiler.job_schedule_profiler_range(3, 2, 5, exit_after_prof=False) is True
    assert profiler.job_schedule_profiler_range(1, 2, 5, exit_after_prof=False) is False
