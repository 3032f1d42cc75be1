"""``paddle.static``: the pieces of the static-graph API that dynamic-to-static capture needs:
``InputSpec`` (python/paddle/static/input.py) and save/load of captured programs."""
from __future__ import annotations

import numpy as np

from .._core import dtype as _dt


class InputSpec:
    def __init__(self, shape=None, dtype="float32", name=None, stop_gradient=False):
        self.shape = tuple(shape) if shape is not None else None
        self.dtype = _dt.to_torch(dtype)
        self.name = name
        self.stop_gradient = stop_gradient

    @classmethod
    def from_tensor(cls, tensor, name=None):
        return cls(list(tensor.shape), tensor.dtype, name or getattr(tensor, "name", None))

    @classmethod
    def from_numpy(cls, ndarray, name=None):
        return cls(ndarray.shape, ndarray.dtype, name)

    def batch(self, batch_size):
        self.shape = (batch_size, *self.shape)
        return self

    def unbatch(self):
        self.shape = self.shape[1:]
        return self

    def matches(self, tensor):
        if self.shape is None:
            return True
        if len(self.shape) != tensor.dim():
            return False
        return all(s is None or s == -1 or s == t for s, t in zip(self.shape, tensor.shape)) and tensor.dtype == self.dtype

    def __repr__(self):
        return f"InputSpec(shape={self.shape}, dtype={_dt.to_name(self.dtype)}, name={self.name})"

    def __hash__(self):
        return hash((self.shape, self.dtype, self.name))

    def __eq__(self, o):
        return isinstance(o, InputSpec) and (self.shape, self.dtype, self.name) == (o.shape, o.dtype, o.name)


def save_inference_model(path_prefix, feed_vars, fetch_vars, executor=None, **kw):
    from ..jit import save
    layer = kw.get("program") or kw.get("layer")
    if layer is None:
        raise ValueError("pass the captured layer as `layer=`")
    save(layer, path_prefix, input_spec=feed_vars)


def load_inference_model(path_prefix, executor=None, **kw):
    from ..jit import load
    return load(path_prefix)


# ======================================================================================= static-graph mode
import contextlib  # noqa: E402
import os  # noqa: E402
import pickle  # noqa: E402

import torch  # noqa: E402

from .._core.tensor import EagerParamBase, as_tensor  # noqa: E402
from . import graph as _g  # noqa: E402
from .graph import (Block, Program, Variable, data, default_main_program, default_startup_program,  # noqa: E402,F401
                    program_guard)


def _plain(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


def _trainable(prog, parameter_list=None, no_grad_set=None):
    params = list(parameter_list) if parameter_list else [p for p in prog.all_parameters() if not p.stop_gradient]
    if params and isinstance(params[0], str):
        params = [prog._find_var(n) for n in params]
    skip = {getattr(v, "name", v) for v in (no_grad_set or ())}
    return [p for p in params if p.name not in skip]


def append_backward(loss, parameter_list=None, no_grad_set=None, callbacks=None, checkpoints=None,
                    distop_context=None):
    """Records the backward pass of ``loss`` (python/paddle/base/backward.py ``append_backward``) and returns
    ``[(param, grad_var)]``; on replay the gradients come from the autograd engine over the replayed forward."""
    prog = default_main_program()
    params = _trainable(prog, parameter_list, no_grad_set)

    def backward(loss_t, *ps):
        grads = torch.autograd.grad(_plain(loss_t), list(ps), retain_graph=True, allow_unused=True)
        return tuple(torch.zeros_like(_plain(p)) if g is None else g for g, p in zip(grads, ps))
    backward._needs_grad = True
    prog._needs_grad = True
    grads = prog.record_py(backward, loss, *params, name="backward")
    out = []
    for p, gr in zip(params, grads):
        gr = as_tensor(gr)
        gr.name = p.name + "@GRAD"
        prog._names[gr.name] = gr
        prog._slot_of_id[id(gr)] = prog._slot_of_key[_g._key(gr)]
        prog._keep.append(gr)
        out.append((p, gr))
    return out


def gradients(targets, inputs, target_gradients=None, no_grad_set=None):
    prog = default_main_program()
    targets = list(targets) if isinstance(targets, (list, tuple)) else [targets]
    inputs = list(inputs) if isinstance(inputs, (list, tuple)) else [inputs]
    tg = list(target_gradients) if isinstance(target_gradients, (list, tuple)) else (
        [target_gradients] if target_gradients is not None else None)
    nt = len(targets)

    def grad_fn(*ts):
        tgt, inp = [_plain(t) for t in ts[:nt]], list(ts[nt:nt + len(inputs)])
        go = [_plain(t) for t in ts[nt + len(inputs):]] or [torch.ones_like(t) for t in tgt]
        gs = torch.autograd.grad(tgt, inp, go, retain_graph=True, allow_unused=True)
        return tuple(torch.zeros_like(i) if g is None else g for g, i in zip(gs, inp))
    grad_fn._needs_grad = True
    prog._needs_grad = True
    outs = prog.record_py(grad_fn, *targets, *inputs, *(tg or []), name="gradients")
    res = []
    for o in outs:
        w = as_tensor(o)
        prog._slot_of_id[id(w)] = prog._slot_of_key[_g._key(w)]
        prog._keep.append(w)
        res.append(w)
    return res


def _static_minimize(opt, loss, parameters=None, no_grad_set=None):
    prog = default_main_program()
    params = _trainable(prog, parameters, no_grad_set)
    if getattr(opt, "_deferred_parameters", False) and not opt._parameter_list:
        opt._set_parameters(params)

    def minimize(loss_t):
        lt = _plain(loss_t)
        if not lt.requires_grad:
            return
        for p in params:
            p.grad = None
        lt.backward()
        opt.step()
    minimize._needs_grad = True
    minimize._train_only = True
    minimize._optimizer, minimize._params = opt, params          # program passes rebuild the step from these
    prog._needs_grad = True
    # the example pass must not move the freshly initialised parameters: record without running
    prog.record(minimize, (loss,), {}, None, name="minimize", inplace=True)
    return None, [(p, None) for p in params]


class _ScopeVar:
    def __init__(self, t):
        self._t = t

    def get_tensor(self):
        return self._t

    def set(self, value, place=None):
        with torch.no_grad():
            _plain(self._t).copy_(torch.as_tensor(value))


class Scope:
    """Name -> persistent tensor lookup (parameters, persistable globals) over every program built so far."""

    def __init__(self):
        self._vars = {}

    def var(self, name):
        v = self.find_var(name)
        if v is None:
            t = as_tensor(torch.empty(0))
            t.name = name
            self._vars[name] = t
            v = _ScopeVar(t)
        return v

    def find_var(self, name):
        if name in self._vars:
            return _ScopeVar(self._vars[name])
        for prog in (_g._S.main, _g._S.startup, *_PROGRAMS, *list(_g.ALL_PROGRAMS)):
            if prog is not None:
                t = prog._find_var(name)
                if t is not None:
                    return _ScopeVar(t)
        return None

    def drop_kids(self):
        pass


_PROGRAMS = []
_scope = Scope()


def global_scope():
    return _scope


@contextlib.contextmanager
def scope_guard(scope):
    global _scope
    prev, _scope = _scope, scope
    try:
        yield
    finally:
        _scope = prev


class BuildStrategy:
    """Attribute bag of executor build options; ``use_cuda_graph`` makes ``CompiledProgram`` replay inference programs
    from a captured CUDA graph."""

    def __init__(self):
        self.use_cuda_graph = False
        self.enable_inplace = True
        self.fuse_elewise_add_act_ops = False
        self.fuse_bn_act_ops = False
        self.fuse_all_optimizer_ops = False
        self.memory_optimize = None
        self.build_cinn_pass = False
        self.sync_batch_norm = False
        self.debug_graphviz_path = ""


class CompiledProgram:
    def __init__(self, program_or_graph, build_strategy=None):
        self._program = program_or_graph
        self._build_strategy = build_strategy or BuildStrategy()
        self._graph = None

    def _run(self, feed, fetch_list):
        prog = self._program
        use_graph = (self._build_strategy.use_cuda_graph and torch.cuda.is_available() and not prog._needs_grad)
        if not use_graph:
            return prog._execute(feed, fetch_list)
        key = tuple((n, tuple(torch.as_tensor(v).shape)) for n, v in sorted(feed.items()))
        if self._graph is None or self._graph[0] != key:
            static_in = {n: torch.as_tensor(v).cuda().clone() for n, v in feed.items()}
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                prog._execute(static_in, fetch_list)
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                outs = prog._execute(static_in, fetch_list)
            self._graph = (key, g, static_in, outs)
        _, g, static_in, outs = self._graph
        for n, v in feed.items():
            static_in[n].copy_(torch.as_tensor(v))
        g.replay()
        return [o.clone() for o in outs]


class Executor:
    """Replays recorded programs (python/paddle/base/executor.py ``Executor.run``)."""

    def __init__(self, place=None):
        self.place = place

    def run(self, program=None, feed=None, fetch_list=None, feed_var_name="feed", fetch_var_name="fetch", scope=None,
            return_numpy=True, use_program_cache=False, use_prune=False):
        prog = program if program is not None else default_main_program()
        compiled = prog if isinstance(prog, CompiledProgram) else None
        if compiled is not None:
            prog = compiled._program
        if prog not in _PROGRAMS:
            _PROGRAMS.append(prog)
        if isinstance(feed, (list, tuple)):
            feed = feed[0] if feed else {}
        feed = feed or {}
        fetch_list = list(fetch_list) if isinstance(fetch_list, (list, tuple)) else ([fetch_list] if fetch_list is not None else [])
        if not prog._nodes and not fetch_list:
            return []                      # startup program: parameters are initialised when they are created
        with _g.suspend():
            outs = compiled._run(feed, fetch_list) if compiled is not None else prog._execute(feed, fetch_list)
            if return_numpy:
                return [o.detach().float().cpu().numpy() if o.dtype == torch.bfloat16 else o.detach().cpu().numpy()
                        for o in outs]
            return [as_tensor(o.detach()) for o in outs]

    def close(self):
        pass

    def train_from_dataset(self, program=None, dataset=None, scope=None, thread=0, debug=False, fetch_list=None,
                           fetch_info=None, print_period=100, fetch_handler=None):
        for batch in dataset:
            self.run(program, feed=batch, fetch_list=fetch_list)

    infer_from_dataset = train_from_dataset


def cpu_places(device_count=None):
    from .. import CPUPlace
    return [CPUPlace()] * (device_count or int(os.environ.get("CPU_NUM", 1)))


def cuda_places(device_ids=None):
    from .. import CUDAPlace
    ids = device_ids if device_ids is not None else range(torch.cuda.device_count())
    return [CUDAPlace(i) for i in ids]


def xpu_places(device_ids=None):
    return []


@contextlib.contextmanager
def name_scope(prefix=None):
    yield


@contextlib.contextmanager
def device_guard(device=None):
    yield


@contextlib.contextmanager
def ipu_shard_guard(index=-1, stage=-1):
    raise RuntimeError("IPU devices are not supported")
    yield


def set_ipu_shard(call_func, index=-1, stage=-1):
    raise RuntimeError("IPU devices are not supported")


class IpuStrategy:
    def __init__(self):
        raise RuntimeError("IPU devices are not supported")


class IpuCompiledProgram:
    def __init__(self, *a, **k):
        raise RuntimeError("IPU devices are not supported")


def create_global_var(shape, value, dtype, persistable=False, force_cpu=False, name=None):
    from .._core import dtype as _dt
    with _g.suspend():
        dev = "cpu" if force_cpu else _dt.default_device()
        t = as_tensor(torch.full([int(s) for s in shape], value, dtype=_dt.to_torch(dtype), device=dev))
    t.persistable = persistable
    if name:
        t.name = name
        default_main_program()._names[name] = t
    return t


def create_parameter(shape, dtype, name=None, attr=None, is_bias=False, default_initializer=None):
    from ..nn.layer.layers import Layer, ParamAttr
    attr = ParamAttr._to_attr(attr)
    if name and attr is not False and attr.name is None:
        attr.name = name
    return Layer().create_parameter(shape, attr, dtype, is_bias, default_initializer)


class WeightNormParamAttr:
    def __new__(cls, dim=None, name=None, initializer=None, learning_rate=1.0, regularizer=None, trainable=True,
                do_model_average=False, need_clip=True):
        from ..nn.layer.layers import ParamAttr
        a = ParamAttr(name=name, initializer=initializer, learning_rate=learning_rate, regularizer=regularizer,
                      trainable=trainable, need_clip=need_clip)
        a.dim = dim
        return a


def Print(input, first_n=-1, message=None, summarize=20, print_tensor_name=True, print_tensor_type=True,
          print_tensor_shape=True, print_tensor_layout=True, print_tensor_lod=True, print_phase="both"):
    def _print(t):
        print(f"{message or ''} shape={list(t.shape)} dtype={t.dtype} data={_plain(t).flatten()[:summarize].tolist()}")
        return t
    if _g.recording():
        return default_main_program().record_py(_print, input, name="print")
    return _print(input)


def py_func(func, x, out, backward_func=None, skip_vars_in_backward_input=None):
    """Runs a Python callable as one op of the program; ``out`` (example variables) is replaced by the results."""
    xs = list(x) if isinstance(x, (list, tuple)) else [x]

    def call(*ts):
        r = func(*ts)
        return r
    if _g.recording():
        return default_main_program().record_py(call, *xs, name="py_func")
    return call(*xs)


def accuracy(input, label, k=1, correct=None, total=None):
    from ..metric import accuracy as _acc
    return _acc(input, label, k)


def auc(input, label, curve="ROC", num_thresholds=4095, topk=1, slide_steps=1, ins_tag_weight=None):
    """Batch AUC from the positive-class probability (column 1 of ``input``)."""
    p = _plain(input)[:, -1].float()
    y = _plain(label).reshape(-1).float()
    order = torch.argsort(p, descending=True)
    y = y[order]
    tp, fp = torch.cumsum(y, 0), torch.cumsum(1 - y, 0)
    tpr = torch.cat([torch.zeros(1), tp / tp[-1].clamp_min(1)])
    fpr = torch.cat([torch.zeros(1), fp / fp[-1].clamp_min(1)])
    val = as_tensor(torch.trapz(tpr, fpr))
    return val, val, []


def ctr_metric_bundle(input, label, ins_tag_weight=None):
    p, y = _plain(input).reshape(-1).float(), _plain(label).reshape(-1).float()
    sqrerr, abserr = ((p - y) ** 2).sum(), (p - y).abs().sum()
    return tuple(as_tensor(t) for t in (sqrerr, abserr, p.sum(), y.sum(), torch.tensor(float(p.numel()))))


class ExponentialMovingAverage:
    """Shadow parameters ``ema = decay * ema + (1 - decay) * param`` with bias correction on ``apply``
    (python/paddle/static/__init__.py exports it from base/optimizer.py)."""

    def __init__(self, decay=0.999, thres_steps=None, name=None):
        self._decay, self._thres, self._name = decay, thres_steps, name
        self._params = [p for p in default_main_program().all_parameters() if not p.stop_gradient]
        with _g.suspend():
            self._ema = [torch.zeros_like(_plain(p)) for p in self._params]
        self._backup, self._step = None, 0

    def update(self):
        if not self._params:
            self._params = [p for p in default_main_program().all_parameters() if not p.stop_gradient]
            with _g.suspend():
                self._ema = [torch.zeros_like(_plain(p)) for p in self._params]

        def ema_update():
            self._step += 1
            d = self._decay if self._thres is None else min(self._decay, (1 + self._step) / (10 + self._step))
            with torch.no_grad():
                for e, p in zip(self._ema, self._params):
                    e.mul_(d).add_(_plain(p).detach(), alpha=1 - d)
            self._last_decay = d
        ema_update._train_only = True
        if _g.recording():
            default_main_program().record(ema_update, (), {}, None, name="ema_update", inplace=True)
        else:
            ema_update()

    @contextlib.contextmanager
    def apply(self, executor=None, need_restore=True):
        with torch.no_grad(), _g.suspend():
            self._backup = [_plain(p).clone() for p in self._params]
            corr = 1.0 - self._decay ** max(self._step, 1)
            for e, p in zip(self._ema, self._params):
                _plain(p).copy_(e / corr)
        try:
            yield
        finally:
            if need_restore:
                self.restore(executor)

    def restore(self, executor=None):
        if self._backup is not None:
            with torch.no_grad(), _g.suspend():
                for b, p in zip(self._backup, self._params):
                    _plain(p).copy_(b)
            self._backup = None


# --------------------------------------------------------------------------------------- persistence
def _persistables(program):
    return {n: v for n, v in program._named_vars() if isinstance(v, EagerParamBase) or getattr(v, "persistable", False)}


def save(program, model_path, protocol=4, **configs):
    d = os.path.dirname(model_path)
    if d:
        os.makedirs(d, exist_ok=True)
    state = {n: _plain(v).detach().cpu().numpy() for n, v in _persistables(program).items()}
    with open(model_path + ".pdparams", "wb") as f:
        pickle.dump(state, f, protocol=protocol)
    with open(model_path + ".pdmodel", "wb") as f:
        f.write(serialize_program([], [], program=program))


def load_program_state(model_path, var_list=None):
    path = model_path if model_path.endswith(".pdparams") else model_path + ".pdparams"
    with open(path, "rb") as f:
        return pickle.load(f)


def set_program_state(program, state_dict):
    mine = _persistables(program)
    with torch.no_grad(), _g.suspend():
        for n, v in state_dict.items():
            if n in mine:
                _plain(mine[n]).copy_(torch.as_tensor(v).reshape(mine[n].shape))


def load(program, model_path, executor=None, var_list=None):
    set_program_state(program, load_program_state(model_path))


def normalize_program(program, feed_vars, fetch_vars, **kwargs):
    p = program.clone(for_test=True)
    p._feed_names = [v.name for v in (feed_vars if isinstance(feed_vars, (list, tuple)) else [feed_vars])]
    p._fetch_slots = [program._slot_of(v) for v in (fetch_vars if isinstance(fetch_vars, (list, tuple)) else [fetch_vars])]
    p._nodes = _g.prune(p._nodes, p._fetch_slots)
    p._stack = [p._nodes]
    return p


def serialize_program(feed_vars, fetch_vars, **kwargs):
    """The program structure (recorded calls, feeds, fetches) without parameter values, as bytes."""
    import cloudpickle
    program = kwargs.get("program") or default_main_program()
    fv = feed_vars if isinstance(feed_vars, (list, tuple)) else [feed_vars]
    tv = fetch_vars if isinstance(fetch_vars, (list, tuple)) else [fetch_vars]
    fetch_slots = [program._slot_of(v) for v in tv]
    nodes = _g.prune(program._nodes, fetch_slots) if fetch_slots else program._nodes
    used = set(_g.block_inputs(nodes)) | set(fetch_slots)
    feed_names = {v.name for v in fv} if fv else set(program._placeholders)
    shell = {"nodes": nodes, "placeholders": {n: (s, tuple(e.shape), e.dtype) for n, (s, e) in program._placeholders.items()
                                              if n in feed_names},
             "captured": {s: (getattr(t, "name", None), tuple(t.shape), t.dtype, isinstance(t, EagerParamBase),
                              None if isinstance(t, EagerParamBase) or getattr(t, "persistable", False) else _plain(t).detach().cpu())
                          for s, t in program._captured.items() if s in used},
             "feed": [v.name for v in fv], "fetch": fetch_slots}
    return cloudpickle.dumps(shell)


def serialize_persistables(feed_vars, fetch_vars, executor=None, **kwargs):
    program = kwargs.get("program") or default_main_program()
    return pickle.dumps({n: _plain(v).detach().cpu().numpy() for n, v in _persistables(program).items()})


def save_to_file(path, content):
    d = os.path.dirname(path)
    if d:
        os.makedirs(d, exist_ok=True)
    with open(path, "wb") as f:
        f.write(content)


def load_from_file(path):
    with open(path, "rb") as f:
        return f.read()


def deserialize_program(data):
    shell = pickle.loads(data)
    p = Program()
    p._nodes = shell["nodes"]
    p._stack = [p._nodes]
    top = 0
    for n, (s, shape, dt) in shell["placeholders"].items():
        ex = as_tensor(torch.zeros(shape, dtype=dt))
        ex.name = n
        p._placeholders[n] = (s, ex)
        p._names[n] = ex
        p._slot_of_id[id(ex)] = s
        p._keep.append(ex)
        top = max(top, s)
    for s, (name, shape, dt, is_param, value) in shell["captured"].items():
        t = value if value is not None else torch.zeros(shape, dtype=dt)
        t = EagerParamBase(t, trainable=False, name=name) if is_param else as_tensor(t)
        if name and not is_param:
            t.name = name
            t.persistable = True
        p._captured[s] = t
        p._slot_of_id[id(t)] = s
        p._keep.append(t)
        top = max(top, s)
    for n in p._nodes:
        top = max([top, *n.out_slots])
    import itertools
    p._slots = itertools.count(top + 1)
    p._for_test = True
    p._feed_names, p._fetch_slots = shell["feed"], shell["fetch"]
    return p


def deserialize_persistables(program, data, executor=None):
    set_program_state(program, pickle.loads(data))


class _FetchHandle:
    """Fetch target of a loaded inference program (resolves to a slot of that program)."""

    def __init__(self, slot):
        self.slot = slot


def save_inference_model(path_prefix, feed_vars, fetch_vars, executor=None, **kw):  # noqa: F811
    layer = kw.get("layer")
    if layer is not None:
        from ..jit import save as _jsave
        return _jsave(layer, path_prefix, input_spec=feed_vars)
    program = kw.get("program") or default_main_program()
    save_to_file(path_prefix + ".pdmodel", serialize_program(feed_vars, fetch_vars, program=program))
    save_to_file(path_prefix + ".pdiparams", serialize_persistables(feed_vars, fetch_vars, executor, program=program))


def load_inference_model(path_prefix, executor=None, **kw):  # noqa: F811
    with open(path_prefix + ".pdmodel", "rb") as f:
        head = f.read()
    try:
        program = deserialize_program(head)
    except Exception:
        from ..jit import load as _jload
        return _jload(path_prefix)
    deserialize_persistables(program, load_from_file(path_prefix + ".pdiparams"), executor)
    fetches = []
    for s in program._fetch_slots:
        h = as_tensor(torch.empty(0))
        program._slot_of_id[id(h)] = s
        program._keep.append(h)
        fetches.append(h)
    return [program, program._feed_names, fetches]


from . import nn  # noqa: E402,F401


from .._core.submodule_alias import alias_submodules as _alias  # noqa: E402
_alias(__name__, ("io", "input", "log_helper", "pir_io"))
_alias(__name__ + ".nn", ("common", "control_flow", "loss", "metric", "sequence_lod", "static_pylayer"))
