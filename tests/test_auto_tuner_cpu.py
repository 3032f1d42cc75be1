"""Auto tuner: search-space enumeration, pruning rules (configuration and history), memory model, recorder,
launcher-argument generation, log reading, resume, and the launcher's tuning loop on a CPU-only toy script
(reference behaviour: python/paddle/distributed/auto_tuner/, test/auto_parallel/test_auto_tuner*.py)."""
import json
import os
import subprocess
import sys
import textwrap

import pytest

from paddle_b200.distributed import auto_tuner as at
from paddle_b200.distributed.auto_tuner import prune, utils
from paddle_b200.distributed.auto_tuner.memory_cost_model import get_model_memory_usage, parse_arguments

MODEL = dict(hidden_size=4096, num_layers=32, num_attention_heads=32, vocab_size=32000, seq_length=4096, global_batch_size=16)


def _cfg(**kw):
    base = dict(num_gpus=8, nodes=1, dp_degree="auto", mp_degree="auto", pp_degree="auto", sharding_degree="auto",
                sharding_stage=[1, 2, 3], micro_batch_size=[1, 2, 4], use_recompute="auto", model_cfg=dict(MODEL))
    base.update(kw)
    return base


def test_candidates_and_search_space():
    cand = at.default_candidates(_cfg())
    assert cand["mp_degree"] == [8, 4, 2, 1] and cand["dp_degree"] == [1, 2, 4, 8] and cand["use_recompute"] == [False, True]
    assert cand["vpp_degree"] == [1] and cand["micro_batch_size"] == [1, 2, 4]
    space = at.search_all(_cfg())
    assert space and all(c["dp_degree"] * c["mp_degree"] * c["pp_degree"] * c["sharding_degree"] == 8 for c in space)
    assert space[0]["pp_degree"] == 1 and space[0]["mp_degree"] == 1 and space[0]["micro_batch_size"] == 4
    two_nodes = at.default_candidates(_cfg(num_gpus=16, nodes=2))
    assert max(two_nodes["mp_degree"]) == 8                         # tensor parallelism stays inside a node


def test_configuration_prunes():
    t = _cfg()
    t["candidates"] = at.default_candidates(t)
    ok = dict(dp_degree=2, mp_degree=4, pp_degree=1, sharding_degree=1, sharding_stage=1, micro_batch_size=2,
              use_recompute=False, vpp_degree=1, global_batch_size=16)
    assert not at.is_pruned(t, dict(ok))
    assert prune.prune_by_mp({**t, "model_cfg": {**MODEL, "num_attention_heads": 6}}, dict(ok))
    assert prune.prune_by_pp(t, {**ok, "pp_degree": 3, "mp_degree": 1})
    assert prune.prune_by_pp(t, {**ok, "vpp_degree": 2})                    # virtual stages without a pipeline
    assert prune.prune_by_vpp(t, {**ok, "pp_degree": 4, "vpp_degree": 3})      # 32 layers over 12 chunks
    assert prune.prune_by_mbs(t, {**ok, "micro_batch_size": 16})
    assert prune.prune_by_mbs(t, {**ok, "dp_degree": 1, "mp_degree": 1, "pp_degree": 8, "micro_batch_size": 4})   # 4 < 8 stages
    assert prune.prune_by_sharding(t, {**ok, "sharding_stage": 2})             # stage 2 with a group of one
    assert prune.prune_by_sharding(t, {**ok, "dp_degree": 1, "mp_degree": 1, "pp_degree": 2, "sharding_degree": 4, "sharding_stage": 3})
    assert prune.prune_by_recompute(t, {**ok, "use_recompute": True, "recompute_granularity": "half"})
    assert prune.prune_by_num_gpus(t, {**ok, "dp_degree": 4})
    assert prune.prune_by_invalid_strategy({**t, "invalid_strategy": ["mp4_pp1"]}, dict(ok))
    assert not prune.prune_by_invalid_strategy({**t, "invalid_strategy": ["mp8_pp1"]}, dict(ok))
    big = {**ok, "dp_degree": 8, "mp_degree": 1, "micro_batch_size": 2}
    assert prune.prune_by_memory_estimation({**t, "max_mem_usage": 80.0}, big) and big["estimated_memory_usage"] > 80
    assert not prune.prune_by_memory_estimation({**t, "memory_estimation_tool": lambda tc, c: 1.0}, dict(big))


def test_history_prunes():
    t = _cfg(metric_cfg={"name": "ips"})
    base = dict(dp_degree=1, mp_degree=2, pp_degree=1, sharding_degree=4, sharding_stage=1, micro_batch_size=2,
                use_recompute=False, vpp_degree=1, global_batch_size=16)
    oom = {**base, "max_mem_usage": "OOM", "ips": None}
    assert prune.prune_by_mbs_history(t, {**base, "micro_batch_size": 4}, [oom])
    assert not prune.prune_by_mbs_history(t, {**base, "micro_batch_size": 1}, [oom])
    assert prune.prune_by_recompute_history(t, {**base, "use_recompute": True}, [{**base, "ips": 10.0}])      # already fits without
    assert prune.prune_by_recompute_history(t, dict(base), [{**base, "use_recompute": True, "max_mem_usage": "OOM"}])
    assert prune.prune_by_sharding_history(t, {**base, "sharding_stage": 2}, [{**base, "ips": 10.0}])
    assert prune.prune_by_sharding_history(t, dict(base), [{**base, "sharding_stage": 2, "error_info": "OOM"}])
    assert prune.prune_by_mp_pp_history(t, {**base, "mp_degree": 1, "dp_degree": 2}, [oom])
    assert not prune.prune_by_mp_pp_history(t, {**base, "mp_degree": 4, "sharding_degree": 2}, [oom])
    assert prune.prune_by_vpp_history(t, {**base, "pp_degree": 2, "mp_degree": 1, "vpp_degree": 4},
                                      [{**base, "pp_degree": 2, "mp_degree": 1, "vpp_degree": 2, "error_info": "OOM"}])

    calls = []

    @at.register_prune
    def never(tuner_cfg, cur_cfg, history):
        calls.append(1)
        return False
    try:
        assert not at.is_pruned(t, dict(base)) and calls
    finally:
        prune._PRUNE_FUNC.remove(never)


def test_memory_model_monotone():
    g = lambda **kw: at.memory_cost_gb(dict(dict(dp_degree=1, mp_degree=1, pp_degree=1, sharding_degree=8, sharding_stage=1,
                                                 micro_batch_size=1, use_recompute=False), **kw), MODEL)
    assert g(sharding_stage=3) < g(sharding_stage=2) < g(sharding_stage=1)
    assert g(micro_batch_size=2) > g() > g(use_recompute=True)
    assert g(mp_degree=8, sharding_degree=1) < g(dp_degree=8, sharding_degree=1)
    # 7B, plain data parallelism: 16 bytes per parameter of state alone is over 100 GB
    assert g(dp_degree=8, sharding_degree=1) > 100
    args = parse_arguments(["--mp_degree", "8", "--num_layers", "32"])
    assert get_model_memory_usage(args) / 2 ** 30 == pytest.approx(g(mp_degree=8, sharding_degree=1), rel=1e-6)
    kept = at.get_not_oom_cfgs(at.search_all(_cfg()), {**_cfg(), "max_mem_usage": 60.0})
    assert kept and all(at.memory_cost_gb(c, MODEL) <= 60.0 for c in kept)


def test_tuner_loop_resume_and_best(tmp_path):
    t = at.AutoTuner(_cfg(task_limit=1000, metric_cfg={"name": "ips", "OptimizationDirection": "max"}))
    seen = []
    while (c := t.search_once()) is not None:
        c = dict(c)
        key = tuple(c[k] for k in ("dp_degree", "mp_degree", "pp_degree", "sharding_degree", "sharding_stage", "micro_batch_size", "use_recompute"))
        assert key not in seen
        seen.append(key)
        oom = c["micro_batch_size"] >= 2 and c["mp_degree"] * c["pp_degree"] <= 2 and not c["use_recompute"]
        c["ips"] = None if oom else 100.0 * c["micro_batch_size"] / (c["mp_degree"] + 2 * c["pp_degree"] + c["use_recompute"])
        c["max_mem_usage"] = "OOM" if oom else 50.0
        t.add_cfg(c)
        if len(seen) == 10:
            t.store_history(str(tmp_path / "h.csv"))
    assert 10 < len(seen) < len(t.candidates)                       # pruning removed part of the space
    best = t.get_best()
    assert best["ips"] == max(h["ips"] for h in t.history_cfgs if h["ips"] is not None)
    # resume: the ten stored trials are not handed out again, and their results count
    t2 = at.AutoTuner(_cfg(task_limit=1000, metric_cfg={"name": "ips", "OptimizationDirection": "max"}))
    assert t2.resume_form_history(str(tmp_path / "h.csv")) and len(t2.resume_cfgs) == 10
    again = []
    while (c := t2.search_once()) is not None:
        again.append(tuple(c[k] for k in ("dp_degree", "mp_degree", "pp_degree", "sharding_degree", "sharding_stage", "micro_batch_size", "use_recompute")))
        c = dict(c)
        oom = c["micro_batch_size"] >= 2 and c["mp_degree"] * c["pp_degree"] <= 2 and not c["use_recompute"]
        c["ips"] = None if oom else 1.0
        c["max_mem_usage"] = "OOM" if oom else 50.0
        t2.add_cfg(c)
    assert not set(again) & set(seen[:10]) and len(again) == len(seen) - 10
    # task limit
    t3 = at.AutoTuner(_cfg(task_limit=3))
    n = 0
    while t3.search_once() is not None:
        n += 1
    assert n == 3
    with pytest.raises(NotImplementedError):
        at.AutoTuner(_cfg(search_algo="annealing"))


def test_other_search_algorithms(tmp_path):
    dp = at.AutoTuner(_cfg(search_algo={"name": "dp_estimation"}, sharding_degree=1, sharding_stage=1))
    c = dp.search_once()
    assert c["dp_degree"] == 1 and c["num_gpus"] * c["estimated_dp_degree"] == 8
    assert c["global_batch_size"] * c["estimated_dp_degree"] == 16
    shapes = {(x["mp_degree"], x["pp_degree"], x["num_gpus"]) for x in dp.candidates}
    assert (8, 1, 8) in shapes and (1, 1, 1) in shapes
    c["ips"] = 5.0
    assert utils.add_overlap_performance(c, {"metric_cfg": {"name": "ips"}}, [])["bw_ips"] == 5.0 * c["estimated_dp_degree"]

    gbs = at.AutoTuner(_cfg(search_algo={"name": "gbs", "max_search_gbs": 64}, dp_degree=1, mp_degree=8, pp_degree=1, sharding_degree=1,
                            sharding_stage=1, micro_batch_size=1, use_recompute=False))
    sizes = []
    while (c := gbs.search_once()) is not None:
        sizes.append(c["global_batch_size"])
        c = dict(c)
        c["ips"], c["max_mem_usage"] = (None, "OOM") if c["global_batch_size"] >= 64 else (1.0, 10.0)
        gbs.add_cfg(c)
    assert sizes == [16, 32, 64]

    csv_path = tmp_path / "mine.csv"
    csv_path.write_text("dp_degree,mp_degree,pp_degree,sharding_degree,micro_batch_size,use_recompute\n"
                        "2,4,1,1,2,false\n1,8,1,1,1,true\n3,1,1,1,1,false\n")
    cu = at.AutoTuner(_cfg(search_algo={"name": "customize", "configs_csv": str(csv_path)}))
    got = []
    while (c := cu.search_once()) is not None:
        got.append((c["dp_degree"], c["mp_degree"], c["use_recompute"]))
        cu.add_cfg({**c, "ips": 1.0})
    assert got == [(2, 4, False), (1, 8, True)]                     # the third row does not multiply to 8 GPUs


def test_recorder_roundtrip(tmp_path):
    r = at.HistoryRecorder({"metric_cfg": {"name": "step_time", "OptimizationDirection": "min"}})
    r.add_cfg(mp_degree=2, step_time=0.5, use_recompute=False, max_mem_usage=170.0)
    r.add_cfg(mp_degree=4, step_time=0.7, use_recompute=True, max_mem_usage=90.0)
    r.add_cfg(mp_degree=8, step_time=None, error_info="OOM")
    best, err = r.get_best()
    assert not err and best["mp_degree"] == 2
    best, _ = r.get_best(buffer=20.0, max_mem_usage=180.0)            # 170 GB is inside the 20 GB safety margin
    assert best["mp_degree"] == 4
    r.store_history(str(tmp_path / "h.csv"))
    r2 = at.HistoryRecorder({})
    rows, missing = r2.load_history(str(tmp_path / "h.csv"))
    assert not missing and rows[0]["step_time"] == 0.5 and rows[1]["use_recompute"] is True and rows[2]["step_time"] is None
    assert at.HistoryRecorder({}).load_history(str(tmp_path / "none.csv")) == ([], True)
    assert at.HistoryRecorder({}).get_best() == (None, True)


def test_gen_new_args_and_logs(tmp_path):
    cfg = dict(dp_degree=2, mp_degree=4, pp_degree=1, sharding_degree=1, micro_batch_size=2, use_recompute=True, global_batch_size=16)
    jpath = tmp_path / "run.json"
    jpath.write_text(json.dumps({"Distributed": {"mp_degree": 1}, "Engine": {}}))
    t = {"run_cmd": {"dp_degree": ["-o", "Distributed.dp_degree"], "micro_batch_size": ["--mbs"],
                     "mp_degree": [str(jpath), "Distributed.mp_degree"], "gradient_accumulation_steps": ["--acc"],
                     "use_recompute": ["--recompute"]}}
    out = at.gen_new_args(["train.py", "-c", str(jpath)], cfg, t)
    assert out[:2] == ["train.py", "-c"] and out[2] != str(jpath) and json.load(open(out[2]))["Distributed"]["mp_degree"] == 4
    rest = out[3:]
    assert rest[rest.index("-o") + 1] == "Distributed.dp_degree=2" and rest[rest.index("--mbs") + 1] == "2"
    assert rest[rest.index("--acc") + 1] == "4" and rest[rest.index("--recompute") + 1] == "True"
    log = tmp_path / "logs"
    log.mkdir()
    (log / "workerlog.0").write_text("".join(f"step {i} loss: 2.0 ips: {100 + i} tokens/s max_memory_allocated: {1000 + i}\n" for i in range(20)))
    val, flag = at.read_metric_log(str(log), target_metric="ips")
    assert flag == 0 and val == pytest.approx(sum(range(110, 120)) / 10)
    assert at.read_metric_log(str(log), target_metric="mfu") == (0.0, 1)
    assert at.read_metric_log(str(tmp_path / "nothing"))[1] == 2
    res = at.read_log(str(log), "workerlog(\\.\\d+)?", "ips")
    assert res["error_info"] is None and res["max_mem_usage"] == 1019.0
    (log / "workerlog.1").write_text("RuntimeError: CUDA out of memory. Tried to allocate 2 GiB\n")
    assert at.find_error_from_log(str(log)) == 1 and at.read_log(str(log), "workerlog(\\.\\d+)?", "ips")["max_mem_usage"] == "OOM"
    (log / "workerlog.1").write_text("Traceback (most recent call last):\n  boom\n")
    assert at.find_error_from_log(str(log)) == 2
    (tmp_path / "mem.csv").write_text("timestamp,memory.used [MiB]\n0,100 MiB\n1,250 MiB\n")
    assert at.read_memory_log(str(tmp_path), "mem.csv") == (250.0, 0)


def test_launcher_auto_tuner_mode(tmp_path):
    """The launcher runs a toy script once per configuration (2 CPU processes each), reads `ips` from its logs, treats
    the script's simulated out-of-memory as such, writes the history and the best configuration."""
    script = tmp_path / "toy.py"
    script.write_text(textwrap.dedent("""
        import argparse, sys
        p = argparse.ArgumentParser()
        p.add_argument("--dp", type=int); p.add_argument("--mp", type=int); p.add_argument("--mbs", type=int)
        a = p.parse_args()
        if a.mbs >= 4:
            print("RuntimeError: CUDA out of memory", flush=True); sys.exit(1)
        for i in range(6):
            print(f"step {i} ips: {100.0 * a.mbs / a.mp}", flush=True)
    """))
    tj = tmp_path / "tune.json"
    tj.write_text(json.dumps({"dp_degree": "auto", "mp_degree": "auto", "pp_degree": 1, "sharding_degree": 1, "micro_batch_size": [1, 2, 4],
                              "use_recompute": False, "task_limit": 20,
                              "model_cfg": {"hidden_size": 64, "num_layers": 2, "num_attention_heads": 2, "vocab_size": 128,
                                            "seq_length": 16, "global_batch_size": 8},
                              "run_cmd": {"dp_degree": ["--dp"], "mp_degree": ["--mp"], "micro_batch_size": ["--mbs"]}}))
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-m", "paddle_b200.distributed.launch", "--nproc_per_node", "2", "--log_dir", str(tmp_path / "log"),
                        "--job_id", "tune", "--poll_interval", "0.05", "--auto_tuner_json", str(tj), str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    best = json.load(open(tmp_path / "log" / "tune_best_cfg.json"))
    assert (best["dp_degree"], best["mp_degree"], best["micro_batch_size"]) == (2, 1, 2) and best["ips"] == pytest.approx(200.0)
    rows, _ = at.HistoryRecorder({}).load_history(str(tmp_path / "log" / "tune_history.csv"))
    assert any(h.get("error_info") == "OOM" for h in rows) and len(rows) >= 3


def test_analytic_cost_model_against_measured_steps_and_tuner_order():
    """The analytic step-time model reproduces the throughputs measured for this repository on B200 (tensor parallel
    Llama-2 7B on 1 / 2 / 4 / 8 GPUs, 13B and 7B with sharding stage 3) within 15 %, behaves monotonically, and drives
    the tuner's trial order."""
    from paddle_b200.cost_model import analytic as A
    m7 = dict(hidden_size=4096, num_layers=32, vocab_size=32000, seq_length=4096, global_batch_size=16, intermediate_size=11008,
              num_attention_heads=32)
    m13 = dict(hidden_size=5120, num_layers=40, vocab_size=32000, seq_length=4096, global_batch_size=32, intermediate_size=13824,
               num_attention_heads=40)
    measured = {1: 23.0e3, 2: 39.6e3, 4: 68.9e3, 8: 94.7e3}                       # tokens / s, bench.py on B200
    for n, want in measured.items():
        est = A.estimate_step_time(m7, dict(dp_degree=1, mp_degree=n, pp_degree=1, sharding_degree=1, micro_batch_size=1))
        assert abs(est.tokens_per_second / want - 1) < 0.15, (n, est.tokens_per_second, want)
    z3 = A.estimate_step_time(m13, dict(mp_degree=1, pp_degree=1, sharding_degree=4, sharding_stage=3, micro_batch_size=1))
    assert abs(z3.tokens_per_second / 38.5e3 - 1) < 0.15 and z3.parts["data_parallel"] > 0.3
    z3b = A.estimate_step_time(m7, dict(mp_degree=1, sharding_degree=2, sharding_stage=3, micro_batch_size=1, global_batch_size=32))
    assert abs(z3b.tokens_per_second / 33.9e3 - 1) < 0.15
    # qualitative behaviour
    e1 = A.estimate_step_time(m7, dict(mp_degree=8, micro_batch_size=1))
    e2 = A.estimate_step_time(m7, dict(mp_degree=8, micro_batch_size=1, use_recompute=True))
    assert e2.seconds > e1.seconds and e2.memory_gb < e1.memory_gb
    pp = A.estimate_step_time(m7, dict(pp_degree=4, mp_degree=2, micro_batch_size=1))
    vpp = A.estimate_step_time(m7, dict(pp_degree=4, mp_degree=2, micro_batch_size=1, vpp_degree=2))
    assert pp.parts["pipeline_bubble"] > vpp.parts["pipeline_bubble"] > 0
    assert A.all_reduce_time(1e9, 8) < A.all_reduce_time(1e9, 2) * 1.2 and A.all_reduce_time(1e9, 16) > 5 * A.all_reduce_time(1e9, 8)
    assert A.matmul_time(4096, 4096, 4096) < A.matmul_time(4096, 4096, 8192) and A.attention_time(1, 4096, 32, 128, backward=True) > \
        A.attention_time(1, 4096, 32, 128)
    assert not A.estimate_step_time(dict(m13, num_layers=80, hidden_size=8192, intermediate_size=28672), dict(micro_batch_size=1)).fits()
    # the tuner tries the estimated-fastest configuration first and skips what cannot fit
    t = at.AutoTuner(_cfg(model_cfg=dict(m7, global_batch_size=64), search_algo={"name": "grid", "sort": "estimated"}, task_limit=5))
    first = t.search_once()
    assert first["estimated_tokens_per_second"] == max(c["estimated_tokens_per_second"] for c in t.candidates)
    assert all(c["estimated_memory_usage"] <= 180 / 1.0737 + 1 for c in t.candidates) and first["mp_degree"] == 1
