"""Program passes (python/paddle/distributed/passes/pass_base.py): a registry of named transformations over
recorded static programs, a context that carries attributes between passes, and a manager that applies a list.

Programs here are recorded call lists (``static.Program``), so a pass is a Python rewrite of that list.  The built-in
passes cover what still has meaning on this runtime: ``fuse_elewise_add_act`` style fusions are done by the kernels
themselves and are registered as no-ops so that strategy files naming them keep working; ``prune_side_effect_free``
drops nodes nothing depends on; ``auto_parallel_recompute`` turns the segments between checkpoints into nodes that
are recomputed in the backward pass; ``auto_parallel_amp`` / ``auto_parallel_fp16`` run the forward under automatic
mixed precision."""
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
           "auto_parallel_sharding", "build_cinn"):
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


class SegmentNode:
    """A run of recorded nodes executed as one node.  ``mode="recompute"``: under autograd the segment runs inside
    ``fleet.recompute`` - only its inputs are kept, the nodes run again in the backward pass.
    ``mode="autocast"``: the nodes run under ``torch.autocast`` with the given dtype."""

    def __init__(self, nodes, in_slots, out_slots, mode, name, dtype=None):
        self.nodes, self.in_slots, self.out_slots, self.mode, self.name = nodes, in_slots, out_slots, mode, name
        self.dtype = dtype
        self.args, self.kwargs, self.func = (), {}, None
        self.runs = 0                                   # times the inner nodes ran (forward + recomputation)

    type = property(lambda self: self.name)

    def run(self, prog, env):
        import torch

        from ...static.graph import _Ref
        ins = [prog._resolve(_Ref(s), env) for s in self.in_slots]

        def body(*vals):
            self.runs += 1
            local = dict(zip(self.in_slots, vals))
            for n in self.nodes:
                n.run(prog, local)
            return tuple(local[s] for s in self.out_slots)
        if self.mode == "autocast":
            dev = next((t.device.type for t in ins if isinstance(t, torch.Tensor)), "cpu")
            with torch.autocast(dev, dtype=self.dtype):
                outs = body(*ins)
        elif torch.is_grad_enabled() and (prog._needs_grad or any(isinstance(t, torch.Tensor) and t.requires_grad for t in ins)):
            from ..fleet.recompute import recompute
            outs = recompute(body, *ins)
            outs = outs if isinstance(outs, (tuple, list)) else (outs,)
        else:
            outs = body(*ins)
        env.update(zip(self.out_slots, outs))

    def __repr__(self):
        return f"{self.out_slots} = {self.name}[{len(self.nodes)} nodes]({self.in_slots})"


def _forward_range(program):
    """Index of the first node that belongs to the backward pass / the optimizer (``len`` when there is none)."""
    for i, n in enumerate(program._nodes):
        if getattr(n.func, "_needs_grad", False) or n.name in ("backward", "gradients", "optimizer_step"):
            return i
    return len(program._nodes)


def _wrap(program, lo, hi, mode, name, keep=(), dtype=None):
    from ...static import graph as g
    nodes = program._nodes[lo:hi]
    produced, used_inside = [], []
    for n in nodes:
        used_inside.extend(s for s in g.node_inputs(n) if s not in produced)
        produced.extend(n.out_slots)
    # captured parameters are passed in too: the recomputation hands their gradients back as input gradients
    in_slots = list(dict.fromkeys(used_inside))
    later = set(g.block_inputs(program._nodes[hi:]))
    named = {program._slot_of_id.get(id(t)) for t in program._names.values()}
    out_slots = [s for s in dict.fromkeys(produced) if s in later or s in named or s in keep]
    if not out_slots:
        out_slots = [produced[-1]]
    program._nodes[lo:hi] = [SegmentNode(nodes, in_slots, out_slots, mode, name, dtype)]


@register_pass("auto_parallel_recompute")
class RecomputePass(PassBase):
    """Recompute instead of keeping activations (python/paddle/distributed/passes/auto_parallel_recompute.py): the
    forward nodes are cut at the variables in attr ``checkpoints`` (variables of the program or their names); every
    segment that ends at a checkpoint becomes one node that keeps only its inputs and runs again during backward.  The
    nodes behind the last checkpoint are left alone.  Attr ``keep``: further variables that must stay fetchable."""

    def _check_self(self):
        return bool(self.get_attr("checkpoints"))

    def _type(self):
        return PassType.CALC_OPT

    def _apply_single_impl(self, main_program, startup_program, context):
        prog = main_program
        cps = [prog._slot_of(v) for v in self.get_attr("checkpoints")]
        keep = {prog._slot_of(v) for v in (self.get_attr("keep") or [])} | set(cps)
        end = _forward_range(prog)
        cuts, start = [], 0
        for i, n in enumerate(prog._nodes[:end]):
            if any(s in cps for s in n.out_slots):
                cuts.append((start, i + 1))
                start = i + 1
        for k, (lo, hi) in enumerate(reversed(cuts)):           # from the back, so that indices stay valid
            if hi - lo >= 2:
                _wrap(prog, lo, hi, "recompute", f"recompute_segment_{len(cuts) - 1 - k}", keep)
        prog._version += 1
        if context is not None:
            context.set_attr("recompute_segments", len(cuts))


@register_pass("auto_parallel_gradient_merge")
class GradientMergePass(PassBase):
    """Accumulate gradients over ``k_steps`` runs of the program and update the parameters on the last of them
    (python/paddle/distributed/passes/auto_parallel_gradient_merge.py).  ``avg`` (default true) divides the sum by
    ``k_steps``.  The recorded ``minimize`` node is rebuilt: runs in between only add to the gradients."""

    def _check_self(self):
        return int(self.get_attr("k_steps", 1) or 1) >= 1

    def _type(self):
        return PassType.CALC_OPT

    def _apply_single_impl(self, main_program, startup_program, context):
        k, avg = int(self.get_attr("k_steps", 1) or 1), bool(self.get_attr("avg", True))
        if k == 1:
            return
        from ...static import _plain
        for node in main_program._nodes:
            f = node.func
            opt, params = getattr(f, "_optimizer", None), getattr(f, "_params", None)
            if node.name != "minimize" or opt is None:
                continue
            state = {"i": 0}

            def merged(loss_t, opt=opt, params=params, state=state):
                lt = _plain(loss_t)
                if not lt.requires_grad:
                    return
                if state["i"] % k == 0:
                    for p in params:
                        p.grad = None
                state["i"] += 1
                (lt / k if avg else lt).backward()
                if state["i"] % k == 0:
                    opt.step()
            merged._needs_grad = merged._train_only = True
            merged._optimizer, merged._params, merged._merge_state = opt, params, state
            node.func = merged
        main_program._version += 1


class _AutocastPass(PassBase):
    """``auto_parallel_amp`` / ``auto_parallel_fp16`` (python/paddle/distributed/passes/auto_parallel_amp.py, _fp16.py):
    the forward nodes run under automatic mixed precision with attr ``dtype`` (``"bfloat16"`` by default for amp on this
    hardware, ``"float16"`` for the fp16 pass).  The cast lists are the runtime's own; ``custom_white_list`` /
    ``custom_black_list`` are accepted and not applied."""
    default_dtype = "bfloat16"

    def _type(self):
        return PassType.CALC_OPT

    def _apply_single_impl(self, main_program, startup_program, context):
        import torch
        dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16}[str(self.get_attr("dtype", self.default_dtype))]
        end = _forward_range(main_program)
        if end:
            keep = {main_program._slot_of(v) for v in (self.get_attr("keep") or [])}
            _wrap(main_program, 0, end, "autocast", "amp_region", keep, dtype)
            main_program._version += 1


register_pass("auto_parallel_amp")(type("AMPPass", (_AutocastPass,), {}))
register_pass("auto_parallel_fp16")(type("FP16Pass", (_AutocastPass,), {"default_dtype": "float16"}))


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
