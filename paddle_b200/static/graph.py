"""Static-graph mode as *record and replay*.

The reference builds a ``Program`` of operator descriptions and interprets it in a C++ executor
(python/paddle/base/framework.py ``Program``/``Block``/``Variable``, python/paddle/base/executor.py ``Executor.run``).
Here the program is a list of recorded tensor-library calls: while static mode is on, every call made between
``paddle.enable_static()`` and ``paddle.disable_static()`` runs once on example data (placeholders declared with
``static.data`` are zero tensors, ``-1``/``None`` dimensions become 1) and is appended to the current ``Program``.
``Executor.run`` replays the list with the fed tensors bound to the placeholders; the replay runs the same eager
kernels (and the autograd engine for ``append_backward`` / ``Optimizer.minimize``), so there is no second
implementation of any operator and a replay can be captured in a CUDA graph (``CompiledProgram``).

Identity of values.  A recorded value is identified by the Python object when it is the object a recorded call
returned, and otherwise by its memory (storage address, offset, sizes, strides, dtype, requires_grad): the framework
functions re-wrap tensors as plain ``torch.Tensor`` aliases before calling the library, and an alias has the same
memory as its source.  All example outputs are kept alive by the program so an address is never reused.
A tensor that reaches a recorded call without having been produced by one is captured by reference (parameters,
buffers, constants); if it carries autograd history it was produced by something the recorder could not see, and the
recorder raises instead of silently baking the example value in.
"""
from __future__ import annotations

import contextlib
import itertools
import weakref

import torch
from torch.overrides import TorchFunctionMode
from torch.utils import _pytree as pytree

from .._core.tensor import EagerParamBase, Tensor, as_tensor


class _Ref:
    __slots__ = ("slot",)

    def __init__(self, slot):
        self.slot = slot

    def __repr__(self):
        return f"%{self.slot}"


def _key(t, with_rg=True):
    if t.numel() == 0 or t.device.type == "meta":
        return ("id", id(t))
    k = (t.untyped_storage().data_ptr(), t.storage_offset(), tuple(t.shape), tuple(t.stride()), t.dtype)
    return k + (t.requires_grad,) if with_rg else k


class Node:
    """One recorded call: ``outs = func(*args, **kwargs)`` with tensors replaced by slot references."""
    __slots__ = ("func", "args", "kwargs", "out_slots", "name")

    def __init__(self, func, args, kwargs, out_slots, name=None):
        self.func, self.args, self.kwargs, self.out_slots = func, args, kwargs, out_slots
        self.name = name or getattr(func, "__name__", None) or str(func)

    def run(self, prog, env):
        res = lambda a: prog._resolve(a, env) if isinstance(a, _Ref) else a       # noqa: E731
        args = pytree.tree_map(res, self.args)
        kwargs = pytree.tree_map(res, self.kwargs)
        if prog._for_test:
            args, kwargs = _eval_mode_args(self.func, args, kwargs)
        try:
            out = self.func(*args, **kwargs)
        except RuntimeError:
            fixed = _repair_baked_shape(self.name, args)
            if fixed is None:
                raise
            out = self.func(*fixed, **kwargs)
        if self.out_slots:
            leaves = [o for o in pytree.tree_leaves(out) if isinstance(o, torch.Tensor)]
            for s, o in zip(self.out_slots, leaves):
                env[s] = o

    @property
    def type(self):
        return self.name

    def __repr__(self):
        return f"{self.out_slots} = {self.name}({self.args}, {self.kwargs})"


def _repair_baked_shape(name, args):
    """Unknown (-1 / None) extents are traced with extent 1, so Python code that turned a shape into integers has
    baked a 1 into ``view`` / ``reshape`` sizes.  When such a call fails at replay because the element count no longer
    matches, the missing factor is put into the first size that was 1 (the batch dimension in practice)."""
    if name not in ("view", "reshape", "_unsafe_view") or len(args) < 2 or not isinstance(args[0], torch.Tensor):
        return None
    sizes = list(args[1]) if isinstance(args[1], (list, tuple, torch.Size)) and len(args) == 2 else list(args[1:])
    if not sizes or not all(isinstance(v, int) for v in sizes) or -1 in sizes or 1 not in sizes:
        return None
    prod = 1
    for v in sizes:
        prod *= v
    numel = args[0].numel()
    if prod == 0 or numel % prod != 0 or numel == prod:
        return None
    sizes[sizes.index(1)] = numel // prod
    return (args[0], sizes)


_TRAIN_FLAG_POS = {}


def _eval_mode_args(func, args, kwargs):
    """A program cloned with ``for_test=True`` runs dropout / batch-norm style calls in inference mode."""
    name = getattr(func, "__name__", "")
    if "training" in kwargs:
        kwargs = dict(kwargs, training=False)
    elif "train" in kwargs:
        kwargs = dict(kwargs, train=False)
    elif name in ("dropout", "alpha_dropout", "feature_alpha_dropout", "dropout1d", "dropout2d", "dropout3d") \
            and len(args) >= 3 and isinstance(args[2], bool):
        args = args[:2] + (False,) + args[3:]
    elif name == "batch_norm" and len(args) >= 6 and isinstance(args[5], bool):
        args = args[:5] + (False,) + args[6:]
    return args, kwargs


def node_inputs(node):
    if hasattr(node, "in_slots"):
        return node.in_slots
    return [a.slot for a in pytree.tree_leaves((node.args, node.kwargs)) if isinstance(a, _Ref)]


def block_inputs(nodes):
    out = []
    for n in nodes:
        out.extend(node_inputs(n))
    return out


def prune(nodes, fetch_slots):
    """The sub-list of ``nodes`` that the fetched values depend on (side-effect-only nodes are dropped)."""
    need, keep = set(fetch_slots), []
    for n in reversed(nodes):
        if any(s in need for s in n.out_slots):
            keep.append(n)
            need.update(node_inputs(n))
    return keep[::-1]


class Block:
    """View of a program's node list with the reference's ``Block`` accessors."""

    def __init__(self, program, nodes, idx=0):
        self.program, self.ops, self.idx = program, nodes, idx

    def var(self, name):
        v = self.program._find_var(name)
        if v is None:
            raise ValueError(f"var {name} is not in this block")
        return v

    def has_var(self, name):
        return self.program._find_var(name) is not None

    def all_parameters(self):
        return self.program.all_parameters()

    @property
    def vars(self):
        return {n: v for n, v in self.program._named_vars()}

    def create_var(self, name=None, shape=None, dtype="float32", persistable=False, **kw):
        from . import create_global_var
        declared = list(shape or [1])
        v = create_global_var([1 if (d is None or d < 0) else int(d) for d in declared], 0.0, dtype, persistable, name=name)
        v._declared_shape = [(-1 if d is None else int(d)) for d in declared]      # unknown extents are recorded as given
        return v


ALL_PROGRAMS = weakref.WeakSet()


class Program:
    _ids = itertools.count()

    def __init__(self):
        self._nodes = []
        self._stack = [self._nodes]
        self._slot_of_id = {}          # id(example tensor) -> slot
        self._slot_of_key = {}         # memory key -> slot
        self._captured = {}            # slot -> tensor captured by reference
        self._keep = []                # example tensors (keeps ids and addresses unique)
        self._placeholders = {}        # name -> (slot, example tensor)
        self._names = {}               # name -> example tensor (named variables)
        self._slots = itertools.count()
        self._for_test = False
        self._needs_grad = False
        self.random_seed = 0
        self._id = next(Program._ids)
        self._version = 0
        ALL_PROGRAMS.add(self)

    # ---------------------------------------------------------------- recording
    def _new_slot(self, t):
        s = next(self._slots)
        self._slot_of_id[id(t)] = s
        self._slot_of_key[_key(t)] = s
        self._keep.append(t)
        return s

    def _slot_for_input(self, t):
        s = self._slot_of_id.get(id(t))
        if s is None:
            s = self._slot_of_key.get(_key(t))
        if s is None and t.requires_grad:
            k = _key(t, False)
            s = self._slot_of_key.get(k + (False,)) if len(k) > 2 else None
        if s is None:
            gf = t.grad_fn
            while gf is not None and type(gf).__name__ == "AliasBackward0":      # plain-tensor alias of ...
                gf = gf.next_functions[0][0] if gf.next_functions else None
            if gf is not None and type(gf).__name__ != "AccumulateGrad":         # ... anything but a leaf
                raise RuntimeError(
                    "static graph: a tensor with autograd history reached a recorded call without having been "
                    f"recorded itself (produced by {type(gf).__name__}); the program cannot be replayed")
            s = next(self._slots)
            self._slot_of_id[id(t)] = s
            self._slot_of_key[_key(t)] = s
            self._captured[s] = t
            self._keep.append(t)
        return s

    def _to_refs(self, obj):
        return pytree.tree_map(lambda a: _Ref(self._slot_for_input(a)) if isinstance(a, torch.Tensor) else a, obj)

    def record(self, func, args, kwargs, out, name=None, inplace=False):
        leaves = [o for o in pytree.tree_leaves(out) if isinstance(o, torch.Tensor)]
        if not leaves and not inplace:
            return
        r_args, r_kwargs = self._to_refs(args), self._to_refs(kwargs or {})
        out_slots = []
        for o in leaves:
            s = self._slot_of_id.get(id(o))
            if s is None:
                s = self._new_slot(o)
            else:                       # an in-place call returned its input: same slot, refreshed value
                self._slot_of_key[_key(o)] = s
            out_slots.append(s)
        self._stack[-1].append(Node(func, r_args, r_kwargs, out_slots, name))
        self._version += 1

    def record_py(self, fn, *args, name=None, **kwargs):
        """Runs ``fn`` now (not recorded internally) and records it as ONE node."""
        with suspend():
            out = fn(*args, **kwargs)
        self.record(fn, args, kwargs, out, name=name or getattr(fn, "__name__", "py_func"), inplace=True)
        return out

    @contextlib.contextmanager
    def _sub_block(self):
        nodes = []
        self._stack.append(nodes)
        try:
            yield nodes
        finally:
            self._stack.pop()

    # ---------------------------------------------------------------- replay
    def _resolve(self, ref, env):
        s = ref.slot
        if s in env:
            return env[s]
        if s in self._captured:
            return self._captured[s]
        raise RuntimeError(f"static graph: value %{s} is used before it is produced (is a fed variable missing?)")

    def _run_nodes(self, nodes, env):
        for n in nodes:
            n.run(self, env)

    def _slot_of(self, var):
        if isinstance(var, str):
            v = self._find_var(var)
            if v is None:
                raise ValueError(f"no variable named {var!r} in the program")
            var = v
        s = self._slot_of_id.get(id(var))
        if s is None:
            s = self._slot_of_key.get(_key(var))
        if s is None:
            raise ValueError("fetch target does not belong to this program")
        return s

    def _execute(self, feed, fetch_list, keep_graph=False):
        """``keep_graph``: fed tensors stay attached to the caller's autograd graph (dy2static replays)."""
        env = {}
        for name, (slot, example) in self._placeholders.items():
            if name in feed:
                v = feed[name]
                t = v.as_subclass(torch.Tensor) if isinstance(v, torch.Tensor) else torch.as_tensor(v)
                t = t.to(device=example.device, dtype=example.dtype)
                if example.requires_grad and not keep_graph:
                    t = t.detach().requires_grad_(True)
                env[slot] = t
        slots = [self._slot_of(v) for v in fetch_list]
        ctx = contextlib.nullcontext() if self._needs_grad else torch.no_grad()
        with suspend(), ctx:
            self._run_nodes(self._nodes, env)
        return [self._resolve(_Ref(s), env) for s in slots]

    # ---------------------------------------------------------------- reference API
    def global_block(self):
        return Block(self, self._nodes)

    def current_block(self):
        return Block(self, self._stack[-1], len(self._stack) - 1)

    def block(self, idx):
        return self.global_block()

    @property
    def blocks(self):
        return [self.global_block()]

    @property
    def num_blocks(self):
        return 1

    def _named_vars(self):
        seen = set()
        for n, v in self._names.items():
            seen.add(n)
            yield n, v
        for t in self._captured.values():
            n = getattr(t, "name", None)
            if n and n not in seen:
                seen.add(n)
                yield n, t

    def _find_var(self, name):
        for n, v in self._named_vars():
            if n == name:
                return v
        return None

    def list_vars(self):
        return [v for _, v in self._named_vars()]

    def all_parameters(self):
        out, seen = [], set()
        for t in self._captured.values():
            if isinstance(t, EagerParamBase) and id(t) not in seen:
                seen.add(id(t))
                out.append(t)
        return out

    def clone(self, for_test=False):
        p = Program.__new__(Program)
        p.__dict__.update(self.__dict__)
        p._nodes = list(self._nodes)
        p._stack = [p._nodes]
        p._for_test = for_test or self._for_test
        if for_test:
            p._nodes = [n for n in p._nodes if not getattr(n.func, "_train_only", False)]
            p._stack = [p._nodes]
            p._needs_grad = any(getattr(n.func, "_needs_grad", False) for n in p._nodes)
        p._id = next(Program._ids)
        ALL_PROGRAMS.add(p)
        return p

    def state_dict(self, mode="all", scope=None):
        return {n: v for n, v in self._named_vars() if isinstance(v, EagerParamBase) or getattr(v, "persistable", False)}

    def set_state_dict(self, state_dict, scope=None):
        mine = self.state_dict()
        with torch.no_grad(), suspend():
            for n, v in state_dict.items():
                if n in mine:
                    mine[n].as_subclass(torch.Tensor).copy_(torch.as_tensor(v.numpy() if hasattr(v, "numpy") else v))

    def to_string(self, throw_on_error=False, with_details=False):
        lines = [f"program #{self._id} ({len(self._nodes)} ops)"]
        lines += [f"  feed {n}: %{s} {tuple(e.shape)}" for n, (s, e) in self._placeholders.items()]
        lines += ["  " + repr(n) for n in self._nodes]
        return "\n".join(lines)

    __str__ = to_string


# -------------------------------------------------------------------- global state
class _State:
    enabled = False
    suspended = 0
    mode = None
    main = None
    startup = None
    orig_apply = None


_S = _State()


def recording():
    return _S.enabled and _S.suspended == 0


def current_program():
    return _S.main


@contextlib.contextmanager
def suspend():
    _S.suspended += 1
    try:
        yield
    finally:
        _S.suspended -= 1


_PASS_THROUGH = {"__get__", "__set__", "__delete__"}


class _Recorder(TorchFunctionMode):
    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if _S.suspended:
            return func(*args, **kwargs)
        name = getattr(func, "__name__", "")
        if name == "backward" and args and isinstance(args[0], torch.Tensor):
            from . import append_backward
            append_backward(args[0])
            return None
        _S.suspended += 1
        try:
            # the example pass must not move running statistics: they belong to the replays
            stats = [(t, t.clone()) for t in args[1:3] if isinstance(t, torch.Tensor)] \
                if name in ("batch_norm", "instance_norm") else ()
            out = func(*args, **kwargs)
            for t, c in stats:
                with torch.no_grad():
                    t.copy_(c)
        finally:
            _S.suspended -= 1
        if name == "__set__" or (name == "__get__" and not isinstance(out, torch.Tensor)):
            return out
        if name in ("__bool__", "__int__", "__float__", "__index__", "item") and args \
                and isinstance(args[0], torch.Tensor) and id(args[0]) in _S.main._slot_of_id:
            import warnings
            warnings.warn(f"static graph: Python read the value of a recorded variable ({name}); the example value is "
                          "baked into the program - use static.nn.cond / while_loop (or to_static(full_graph=True)) "
                          "for data-dependent control flow", stacklevel=3)
        inplace = name.endswith("_") and not name.endswith("__")
        _S.main.record(func, args, kwargs, out, inplace=inplace)
        return out


def _patched_apply(cls, *args, **kwargs):
    if not recording():
        return _S.orig_apply(cls, *args, **kwargs)
    with suspend():
        out = _S.orig_apply(cls, *args, **kwargs)
    _S.main.record(cls.apply, args, kwargs, out, name=cls.__name__)
    return out


def enable():
    if _S.enabled:
        return
    if _S.main is None:
        _S.main, _S.startup = Program(), Program()
    _S.orig_apply = torch.autograd.Function.apply.__func__
    torch.autograd.Function.apply = classmethod(_patched_apply)
    _S.mode = _Recorder()
    _S.mode.__enter__()
    _S.enabled = True


def disable():
    if not _S.enabled:
        return
    _S.mode.__exit__(None, None, None)
    torch.autograd.Function.apply = classmethod(_S.orig_apply)
    _S.mode = None
    _S.enabled = False


def no_trace(fn):
    """Decorator: the call is executed but not recorded (layer construction, parameter initialisation)."""
    import functools

    @functools.wraps(fn)
    def wrapper(*a, **k):
        if not _S.enabled or _S.suspended:
            return fn(*a, **k)
        _S.suspended += 1
        try:
            return fn(*a, **k)
        finally:
            _S.suspended -= 1
    return wrapper


@contextlib.contextmanager
def program_guard(main_program, startup_program=None):
    prev = (_S.main, _S.startup)
    _S.main = main_program
    if startup_program is not None:
        _S.startup = startup_program
    try:
        yield
    finally:
        _S.main, _S.startup = prev


def default_main_program():
    if _S.main is None:
        _S.main, _S.startup = Program(), Program()
    return _S.main


def default_startup_program():
    default_main_program()
    return _S.startup


def data(name, shape, dtype=None, lod_level=0):
    """Declares a fed variable; the example tensor is zeros with unknown (-1 / None) extents set to 1."""
    from .._core import dtype as _dt
    prog = default_main_program()
    ex_shape = [1 if (s is None or s < 0) else int(s) for s in shape]
    with suspend():
        t = as_tensor(torch.zeros(ex_shape, dtype=_dt.to_torch(dtype or "float32"), device=_dt.default_device()))
        t.stop_gradient = True
    t.name = name
    t.persistable = False
    t._declared_shape = [(-1 if s is None else int(s)) for s in shape]
    slot = prog._new_slot(t)
    prog._placeholders[name] = (slot, t)
    prog._names[name] = t
    return t


Variable = Tensor
