"""Program passes (python/paddle/distributed/passes/pass_base.py): a registry of named transformations over
recorded static programs, a context that carries attributes between passes, and a manager that applies a list.

Programs here are recorded call lists (``static.Program``), so a pass is a Python rewrite of that list.  The built-in
passes cover what still has meaning on this runtime: ``fuse_elewise_add_act`` style fusions are done by the kernels
themselves and are registered as no-ops so that strategy files naming them keep working; ``prune_side_effect_free``
drops nodes nothing depends on."""
from __future__ import annotations


class PassContext:
    def __init__(self):
        self._applied_passes, self._attrs = [], {}

    def set_attr(self, key, value):
        self._attrs[key] = value

    def get_attr(self, key, default=None):
        return self._attrs.get(key, default)

    @property
    def passes(self):
        return self._applied_passes

    def _add_pass(self, p):
        self._applied_passes.append(p)

    def _pop_pass(self):
        del self._applied_passes[-1]


class PassType:
    UNKNOWN, COMM_OPT, CALC_OPT, PARALLEL_OPT, FUSION_OPT = 0, 1, 2, 3, 4


class PassBase:
    _REGISTERED_PASSES = {}
    name = None

    def __init__(self):
        self._attrs = {}

    def set_attr(self, key, value):
        self._attrs[key] = value
        return self

    def get_attr(self, key, default=None):
        return self._attrs.get(key, default)

    def _check_self(self):
        return True

    def _check_conflict(self, other_pass):
        return True

    def _type(self):
        return PassType.UNKNOWN

    def apply(self, main_programs, startup_programs, context=None):
        context = context or PassContext()
        if not self._check_self() or not all(self._check_conflict(p) for p in context.passes):
            return context
        mains = main_programs if isinstance(main_programs, (list, tuple)) else [main_programs]
        starts = startup_programs if isinstance(startup_programs, (list, tuple)) else [startup_programs] * len(mains)
        for m, s in zip(mains, starts):
            self._apply_single_impl(m, s, context)
        context._add_pass(self)
        return context

    def _apply_single_impl(self, main_program, startup_program, context):
        raise NotImplementedError


def register_pass(name):
    def deco(cls):
        cls.name = name
        PassBase._REGISTERED_PASSES[name] = cls
        return cls
    return deco


def new_pass(name, pass_attrs={}):
    cls = PassBase._REGISTERED_PASSES.get(name)
    assert cls is not None, f"Pass {name} is not registered"
    p = cls()
    for k, v in pass_attrs.items():
        p.set_attr(k, v)
    return p


class PassManager:
    def __init__(self, passes, context=None, auto_solve_conflict=True):
        self._context = context or PassContext()
        self._passes = list(passes)

    def apply(self, main_programs, startup_programs):
        for p in self._passes:
            self._context = p.apply(main_programs, startup_programs, self._context)
        return self._context

    @property
    def context(self):
        return self._context

    @property
    def names(self):
        return [p.name for p in self._passes]


class _NoOp(PassBase):
    def _apply_single_impl(self, main_program, startup_program, context):
        pass


for _n in ("fuse_elewise_add_act", "fuse_bn_act", "fuse_bn_add_act", "fuse_relu_depthwise_conv", "fuse_optimizer",
           "fuse_all_reduce", "fuse_gemm_epilogue", "fused_attention", "fused_feedforward", "inplace_addto_op",
           "auto_parallel_amp", "auto_parallel_fp16", "auto_parallel_recompute", "auto_parallel_sharding",
           "auto_parallel_gradient_merge", "build_cinn"):
    register_pass(_n)(type(f"_{_n}", (_NoOp,), {}))


@register_pass("prune_side_effect_free")
class PruneSideEffectFree(PassBase):
    """Keeps only the nodes that the program's named fetch targets (attr ``fetch``) depend on."""

    def _apply_single_impl(self, main_program, startup_program, context):
        from ...static import graph as g
        targets = self.get_attr("fetch", [])
        if not targets:
            return
        slots = [main_program._slot_of(t) for t in targets]
        main_program._nodes[:] = g.prune(main_program._nodes, slots)


class _PipelineSchedulerPass(PassBase):
    """``pipeline_scheduler_<mode>``: the reference rewrites a program into per-micro-batch jobs
    (python/paddle/distributed/passes/pipeline_scheduler_pass/); here the job list is the generated step list of
    ``fleet/meta_parallel/pipeline_schedules.py``, returned in ``context`` under ``"job_list"`` after validation."""
    mode = "1F1B"

    def _apply_single_impl(self, main_program, startup_program, context):
        from ..fleet.meta_parallel import pipeline_schedules as S
        P, M = int(self.get_attr("pp_degree")), int(self.get_attr("num_micro_batches"))
        V = int(self.get_attr("vpp_degree") or 1)
        fn = S.SCHEDULES[self.mode]
        S.validate(fn, P, V, M)
        jobs = fn(P, V, M, int(self.get_attr("pp_stage") or 0))
        if context is not None:
            context.set_attr("job_list", jobs)
        return jobs


for _mode in ("FThenB", "1F1B", "VPP", "ZBH1"):
    register_pass(f"pipeline_scheduler_{_mode}")(type(f"PipelineScheduler{_mode}", (_PipelineSchedulerPass,), {"mode": _mode}))
