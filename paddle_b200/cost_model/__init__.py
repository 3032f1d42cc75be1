"""``paddle.cost_model.CostModel`` (python/paddle/cost_model/cost_model.py): measured per-operator cost of a static
program.  ``profile_measure`` replays the program once with each recorded call timed (CUDA events on GPU, wall clock
on CPU) and returns ``{op name: {"calls": n, "time_ms": t}}``; ``static_cost_data`` / ``get_static_op_time`` serve the
table of the last measurement."""
from __future__ import annotations

import time

import torch

from . import analytic  # noqa: E402,F401
from .analytic import Cluster, estimate_step_time, rank_configs  # noqa: E402,F401

__all__ = ["CostModel"]


class CostModel:
    def __init__(self):
        self._table = {}

    def build_program(self):
        from .. import static
        import paddle_b200 as paddle
        main, startup = static.Program(), static.Program()
        with static.program_guard(main, startup):
            data = static.data("X", [None, 1], "float32")
            hidden = static.nn.fc(data, 10)
            loss = paddle.mean(hidden)
            paddle.optimizer.SGD(learning_rate=0.01).minimize(loss)
        return startup, main

    def profile_measure(self, startup_program, main_program, device="gpu", fetch_cost_list=("time",), feed=None):
        from ..static import graph as g
        use_cuda = device == "gpu" and torch.cuda.is_available()
        env, table = {}, {}
        feed = feed or {}
        for name, (slot, ex) in main_program._placeholders.items():
            t = torch.as_tensor(feed[name]) if name in feed else ex.as_subclass(torch.Tensor).clone()
            env[slot] = t.to(ex.device)
        with g.suspend():
            for node in main_program._nodes:
                if use_cuda:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    node.run(main_program, env)
                    e1.record()
                    e1.synchronize()
                    ms = e0.elapsed_time(e1)
                else:
                    t0 = time.perf_counter()
                    node.run(main_program, env)
                    ms = (time.perf_counter() - t0) * 1e3
                rec = table.setdefault(node.name, {"calls": 0, "time_ms": 0.0})
                rec["calls"] += 1
                rec["time_ms"] += ms
        self._table = table
        return table

    def static_cost_data(self):
        return self._table

    def get_static_op_time(self, op_name, forward=True, dtype="float32"):
        rec = self._table.get(op_name)
        if rec is None:
            raise ValueError(f"op {op_name!r} has not been measured; call profile_measure first")
        return {"op_time": rec["time_ms"] / max(rec["calls"], 1), "config": {"dtype": dtype, "forward": forward}}
