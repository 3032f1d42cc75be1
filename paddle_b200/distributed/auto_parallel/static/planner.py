"""Search for a parallel plan of a recorded program (the role of python/paddle/distributed/auto_parallel/static/
planner_v2.py with tuner/rule_based_tuner.py and tuner/parallel_tuner.py).

For every factorisation of the device count into a (data, tensor) mesh the planner tries a few annotation strategies,
completes each with the SPMD rules, prices it with the cost estimator and keeps the fastest plan that fits the device
memory:

* ``dp``: the batch dim of every data input is split over the data axis; nothing else is annotated.
* ``mp``: in addition, every weight of a matmul / linear whose activation input does not already carry the tensor axis on
  its contracted dim is split by output features (column parallel).  Completion then does the rest: the next weight
  on the path meets an activation whose contracted dim is split and adopts the matching row split, its output is a
  partial sum that is all-reduced where a consumer needs the whole value; a projection that feeds a cross entropy keeps
  the class dim split (the vocabulary-parallel loss).
* ``mp+vocab``: embedding tables are split by rows (vocabulary) as well.
* ``mp+sp``: like ``mp``, and the sequence dim (dim 1) of the data is split over the tensor axis too, so that everything
  between the parallel products - normalisation, residual adds, dropout - works on a sequence slice: completion puts an
  all-gather in front of each column-parallel product and turns the all-reduce behind each row-parallel one into a
  reduce-scatter (Megatron sequence parallelism).

A column split is dropped again when it makes the plan slower than leaving that weight whole (a greedy pass over the
candidates, costliest re-shards first), so a weight whose output is needed whole right away stays replicated."""
from __future__ import annotations

from dataclasses import dataclass, field

from .completion import Completer
from .cost import CostEstimator


@dataclass
class Plan:
    mesh_shape: list
    dim_names: list
    strategy: str
    annotations: dict                       # slot -> dims_mapping fixed before completion
    cost: object = None
    parts: dict = field(default_factory=dict)
    dist_context: object = None

    def param_specs(self):
        """``{parameter: dims_mapping}`` for every parameter of the program."""
        c = self.dist_context
        return {t: list(c.tensor_specs[s].dims_mapping) for s, t in c.params.items() if s in c.tensor_specs}

    def placements(self, tensor):
        """The ``Shard`` / ``Replicate`` list of a parameter for ``shard_tensor``."""
        from ..process_mesh import Replicate, Shard
        c = self.dist_context
        for s, t in c.params.items():
            if t is tensor:
                pl = [Replicate()] * len(self.mesh_shape)
                for d, m in enumerate(c.tensor_specs[s].dims_mapping):
                    if m != -1:
                        pl[m] = Shard(d)
                return pl
        raise KeyError("the tensor is not a parameter of the planned program")

    def process_mesh(self):
        import numpy as np

        from ..process_mesh import ProcessMesh
        n = 1
        for s in self.mesh_shape:
            n *= s
        return ProcessMesh(np.arange(n).reshape(self.mesh_shape).tolist(), self.dim_names)

    def apply(self, layer=None):
        """Shard the parameters the way the plan says (each rank keeps its piece); returns the process mesh."""
        from ..api import shard_tensor
        mesh = self.process_mesh()
        c = self.dist_context
        for s, t in c.params.items():
            if s not in c.tensor_specs:
                continue
            d = shard_tensor(t, mesh, self.placements(t))
            if layer is not None:
                for sub in layer.sublayers(include_self=True):
                    for k, p in list(sub._parameters.items()):
                        if p is t:
                            sub._parameters[k] = d
        return mesh

    def __repr__(self):
        return f"Plan(mesh={dict(zip(self.dim_names, self.mesh_shape))}, strategy={self.strategy!r}, cost={self.cost})"


def _factorisations(n):
    return [(d, n // d) for d in range(1, n + 1) if n % d == 0]


class Planner:
    def __init__(self, program, cluster=None, n_devices=None, mode="train", memory_limit=None, batch_dim=0,
                 mesh_candidates=None, strategies=("dp", "mp", "mp+vocab", "mp+sp"), refine=True, seq_dim=1, assume_dtype=None):
        from .cluster import get_default_cluster
        self.program, self.mode = program, mode
        if cluster is None:
            cluster = get_default_cluster(device_count=n_devices)
        self.cluster = cluster
        self.n_devices = n_devices or len(cluster.get_all_devices("GPU"))
        gpus = cluster.get_all_devices("GPU")
        self.memory_limit = memory_limit if memory_limit is not None else (gpus[0].memory * 1e9 * 0.92 if gpus else float("inf"))
        self.batch_dim, self.seq_dim = batch_dim, seq_dim
        self.assume_dtype = assume_dtype
        self.mesh_candidates = mesh_candidates or _factorisations(self.n_devices)
        self.strategies, self.refine = tuple(strategies), refine
        self.trials = []

    # ---------------------------------------------------------------- annotation strategies
    def _data_annotations(self, comp, dp, sp=1):
        out = {}
        for name, s in comp.ctx.placeholders.items():
            shp = comp.ctx.shapes[s]
            m = [-1] * len(shp)
            if dp > 1 and len(shp) > self.batch_dim and shp[self.batch_dim] % dp == 0:
                m[self.batch_dim] = 0
            if sp > 1 and len(shp) > self.seq_dim and shp[self.seq_dim] % sp == 0:
                m[self.seq_dim] = 1
            if any(v != -1 for v in m):
                out[s] = m
        return out

    def _evaluate(self, mesh, annotations, strategy):
        comp = Completer(self.program, list(mesh), ["dp", "mp"], assume_dtype=self.assume_dtype)
        if strategy.endswith("+sp"):
            comp.prefer_scatter = {1: self.seq_dim}
        for s, m in annotations.items():
            comp.annotate(s, m)
        ctx = comp.complete_forward_annotation()
        est = CostEstimator(ctx, self.cluster, self.mode)
        cost = est.estimate_cost()
        return Plan(list(mesh), ["dp", "mp"], strategy, dict(annotations), cost, dict(est.parts), ctx), est

    def _column_candidates(self, mesh, annotations, vocab, seq_parallel=False):
        """One completion pass that adds a column split to every weight whose activation input does not carry the tensor
        axis yet, at the moment the operator is reached (-> all annotations, the slots that were added)."""
        from .completion import _refs
        mp = mesh[1]
        added = []
        comp = Completer(self.program, list(mesh), ["dp", "mp"], assume_dtype=self.assume_dtype)
        for s, m in annotations.items():
            comp.annotate(s, m)

        def hook(c, node):
            name = node.name
            if name not in ("matmul", "mm", "linear", "conv2d", "embedding"):
                return
            refs = _refs((node.args, node.kwargs))
            if len(refs) < 2:
                return
            x_slot, w_slot = refs[0].slot, refs[1].slot
            if w_slot not in c.ctx.params or w_slot in c._annotated:
                return
            w_shape = c.ctx.shapes[w_slot]
            if name == "embedding":
                if vocab and w_shape[0] % mp == 0:
                    c._annotated[w_slot] = [1, -1]
                    added.append(w_slot)
                return
            xm = c._spec(x_slot).dims_mapping
            if len(w_shape) < 2 or not xm or xm[-1] == 1 or (1 in xm and not seq_parallel):
                return
            out_dim = 0 if name in ("linear", "conv2d") else len(w_shape) - 1
            if w_shape[out_dim] % mp == 0 and w_shape[out_dim] >= mp:
                m = [-1] * len(w_shape)
                m[out_dim] = 1
                c._annotated[w_slot] = m
                added.append(w_slot)
        comp.pre_op_hook = hook
        if seq_parallel:
            comp.prefer_scatter = {1: self.seq_dim}
        comp.complete_forward_annotation()
        return dict(comp._annotated), added

    # ---------------------------------------------------------------- search
    def plan(self):
        best = None
        self.trials = []
        for mesh in self.mesh_candidates:
            dp, mp = mesh
            probe = Completer(self.program, list(mesh), ["dp", "mp"], assume_dtype=self.assume_dtype)
            data = self._data_annotations(probe, dp)
            if dp > 1 and not any(0 in m for m in data.values()):
                continue                                            # nothing to split the batch of
            for strategy in self.strategies:
                if strategy != "dp" and mp == 1:
                    continue
                if strategy == "dp" and mp > 1:
                    continue                                        # idle tensor axis: dominated by (dp * mp, 1)
                ann = dict(data)
                added = []
                if strategy != "dp":
                    sp = strategy.endswith("+sp")
                    base = self._data_annotations(probe, dp, mp) if sp else data
                    if sp and base == data:
                        continue                                    # no sequence dim to split
                    ann, added = self._column_candidates(mesh, base, vocab=strategy.endswith("vocab"), seq_parallel=sp)
                    if not added:
                        continue
                plan, est = self._evaluate(mesh, ann, strategy)
                if self.refine and added:
                    plan = self._refine(mesh, plan, added, base if strategy != "dp" else data, strategy)
                fits = plan.cost.memory <= self.memory_limit
                self.trials.append({"mesh": list(mesh), "strategy": strategy, "time": plan.cost.time, "memory": plan.cost.memory,
                                    "fits": fits, "parts": plan.parts})
                if fits and (best is None or plan.cost.time < best.cost.time):
                    best = plan
        if best is None:
            raise RuntimeError("no plan fits the device memory; trials: " + repr([(t["mesh"], t["strategy"], t["memory"]) for t in self.trials]))
        return best

    def _refine(self, mesh, plan, added, data, strategy):
        """Drop a column split when the plan is faster without it (one pass, weights in program order)."""
        for s in added:
            if s not in plan.annotations:
                continue
            trial_ann = {k: v for k, v in plan.annotations.items() if k != s}
            # weights downstream may have been annotated because of ``s``: rebuild those choices
            kept = {k: v for k, v in trial_ann.items() if k in data or k in added}
            trial, _ = self._evaluate(mesh, kept, strategy)
            if trial.cost.time < plan.cost.time * 0.999 and trial.cost.memory <= max(self.memory_limit, plan.cost.memory):
                plan = trial
        return plan


class RuleBasedTuner(Planner):
    """Name of the reference's pattern-driven tuner (tuner/rule_based_tuner.py); ``tune()`` returns the best plan."""

    def tune(self):
        return self.plan()


class ParallelTuner(RuleBasedTuner):
    pass
