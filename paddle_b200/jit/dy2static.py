"""Dynamic-to-static conversion of Python control flow (python/paddle/jit/dy2static/: ``IfElseTransformer``,
``LoopTransformer``, ``LogicalTransformer`` and the ``convert_ifelse`` / ``convert_while_loop`` /
``convert_logical_*`` run-time helpers).

``convert_function`` rewrites a function's source so that every ``if`` / ``while`` whose test may be a tensor goes
through a helper:

    if t: A else: B        ->  def true_fn(): nonlocal v..; A        def false_fn(): nonlocal v..; B
                               v.. = _jst.convert_ifelse(t, true_fn, false_fn, get_args, set_args, names)
    while t: A             ->  v.. = _jst.convert_while(cond_fn, body_fn, get_args, set_args, names)
    a and b / not a        ->  _jst.and_(lambda: a, lambda: b) / _jst.not_(a)

The helpers keep plain Python semantics when the test is a Python value or no static program is being recorded, and
emit ``static.nn.cond`` / ``static.nn.while_loop`` nodes (both branches traced, selected at replay) when the test is
a tensor under static recording.  ``ProgramFunction`` is the ``to_static(full_graph=True)`` callable: it records the
converted function into a ``static.Program`` once per input signature and replays the program afterwards, with
autograd flowing through the replay to the inputs and captured parameters.

A ``return`` that ends a branch of an ``if`` is lifted first (``__jst_ret = value`` in the branch, the statements after
the ``if`` move into its ``else``, one ``return __jst_ret`` at the end).  Limits: any other ``if`` / ``while`` that
contains ``return`` / ``break`` / ``continue`` / ``yield`` is left as Python control flow (its test must then be a
Python value at trace time); variables assigned in only one branch must not be
read afterwards when the other branch ran."""
from __future__ import annotations

import ast
import functools
import inspect
import textwrap

import torch

from .._core.tensor import as_tensor


class _Undefined:
    def __repr__(self):
        return "<undefined>"


UNDEF = _Undefined()


def ld(thunk):
    try:
        return thunk()
    except NameError:
        return UNDEF


def _recording():
    from ..static import graph
    return graph.recording()


def _is_traced_pred(p):
    return isinstance(p, torch.Tensor) and _recording()


def _truth(p):
    if isinstance(p, torch.Tensor):
        return bool(p.as_subclass(torch.Tensor).reshape(-1)[0].item()) if p.numel() == 1 else bool(p.all())
    return bool(p)


def and_(*thunks):
    val = thunks[0]()
    for t in thunks[1:]:
        if isinstance(val, torch.Tensor) and _recording():
            import paddle_b200 as paddle
            nxt = t()
            val = paddle.logical_and(val, nxt if isinstance(nxt, torch.Tensor) else as_tensor(torch.as_tensor(nxt)))
            continue
        if not _truth(val):
            return val
        val = t()
    return val


def or_(*thunks):
    val = thunks[0]()
    for t in thunks[1:]:
        if isinstance(val, torch.Tensor) and _recording():
            import paddle_b200 as paddle
            nxt = t()
            val = paddle.logical_or(val, nxt if isinstance(nxt, torch.Tensor) else as_tensor(torch.as_tensor(nxt)))
            continue
        if _truth(val):
            return val
        val = t()
    return val


def range_cond(i, stop, step):
    """Loop test of a converted ``for .. in range``: a tensor step is assumed positive."""
    descending = not isinstance(step, torch.Tensor) and step < 0
    return i > stop if descending else i < stop


def not_(x):
    if isinstance(x, torch.Tensor) and _recording():
        import paddle_b200 as paddle
        return paddle.logical_not(x)
    return not _truth(x)


def convert_ifelse(pred, true_fn, false_fn, get_args, set_args, names):
    if not _is_traced_pred(pred):
        (true_fn if _truth(pred) else false_fn)()
        return get_args()
    from ..static import nn as snn
    start = get_args()

    def run(fn):
        def branch():
            set_args(start)
            fn()
            return list(get_args())
        return branch
    # first find out which variables are tensors in both branches (only those can be selected at run time)
    t_vals, f_vals = run(true_fn)(), run(false_fn)()
    for n, a, b in zip(names, t_vals, f_vals):
        ta, tb = isinstance(a, torch.Tensor), isinstance(b, torch.Tensor)
        if ta != tb and not (a is UNDEF or b is UNDEF):
            raise TypeError(f"'{n}' is a tensor in one branch of a tensor-dependent `if` and {type(b if ta else a).__name__} "
                            "in the other")
        if not ta and not tb and a is not UNDEF and b is not UNDEF and a != b:
            raise TypeError(f"'{n}' takes different Python values ({a!r} / {b!r}) in the branches of a tensor-dependent "
                            "`if`; make it a tensor")
    sel = [i for i, (a, b) in enumerate(zip(t_vals, f_vals)) if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor)]
    # the probe runs above were recorded too; they are dead code that pruning removes, the cond node re-traces them
    outs = snn.cond(pred, lambda: [run(true_fn)()[i] for i in sel], lambda: [run(false_fn)()[i] for i in sel])
    result = [a if a is not UNDEF else b for a, b in zip(t_vals, f_vals)]
    for i, o in zip(sel, outs or []):
        result[i] = o
    set_args(tuple(result))
    return tuple(result)


def convert_while(cond_fn, body_fn, get_args, set_args, names):
    pred = cond_fn()
    if not _is_traced_pred(pred):
        while _truth(pred):
            body_fn()
            pred = cond_fn()
        return get_args()
    import paddle_b200 as paddle
    from ..static import nn as snn
    start = list(get_args())
    # Python numbers carried by the loop become tensors so that they can change between iterations
    for i, v in enumerate(start):
        if isinstance(v, bool):
            continue
        if isinstance(v, (int, float)):
            start[i] = paddle.to_tensor(v)
    idx = [i for i, v in enumerate(start) if isinstance(v, torch.Tensor)]

    def put(vals):
        cur = list(start)
        for i, v in zip(idx, vals):
            cur[i] = v
        set_args(tuple(cur))

    def c(*vals):
        put(vals)
        return cond_fn()

    def b(*vals):
        put(vals)
        body_fn()
        after = get_args()
        return [after[i] for i in idx]
    outs = snn.while_loop(c, b, [start[i] for i in idx])
    put(outs)
    return get_args()


# ----------------------------------------------------------------------------------------- AST rewriting
def _assigned_names(nodes):
    names = []

    class V(ast.NodeVisitor):
        def visit_Name(self, n):
            if isinstance(n.ctx, (ast.Store, ast.Del)) and n.id not in names:
                names.append(n.id)

        def visit_FunctionDef(self, n):      # nested definitions have their own scope
            if n.name not in names:
                names.append(n.name)

        visit_AsyncFunctionDef = visit_FunctionDef

        def visit_Lambda(self, n):
            pass

        def visit_ListComp(self, n):
            pass

        visit_SetComp = visit_DictComp = visit_GeneratorExp = visit_ListComp
    for n in nodes:
        V().visit(n)
    return [n for n in names if not n.startswith("__jst_") or n.startswith("__jst_i_") or n == "__jst_ret"]


def _has_jump(nodes):
    class V(ast.NodeVisitor):
        found = False

        def visit_Return(self, n):
            self.found = True

        visit_Break = visit_Continue = visit_Yield = visit_YieldFrom = visit_Return

        def visit_FunctionDef(self, n):
            pass

        visit_AsyncFunctionDef = visit_Lambda = visit_FunctionDef
    v = V()
    for n in nodes:
        v.visit(n)
    return v.found


def _parse_stmt(src):
    return ast.parse(textwrap.dedent(src)).body


class _Transformer(ast.NodeTransformer):
    def __init__(self):
        self.k = 0

    def _uid(self):
        self.k += 1
        return self.k

    def _accessors(self, uid, names):
        tup = ", ".join(names) + ("," if len(names) == 1 else "")
        code = f"""
def __jst_get_{uid}():
    return ({tup})
def __jst_set_{uid}(__jst_v):
    nonlocal {", ".join(names)}
    ({tup}) = __jst_v
"""
        return _parse_stmt(code)

    def _prelude(self, names):
        return [_parse_stmt(f"{n} = _jst.ld(lambda: {n})")[0] for n in names]

    def visit_BoolOp(self, node):
        self.generic_visit(node)
        fn = "and_" if isinstance(node.op, ast.And) else "or_"
        args = [ast.Lambda(args=ast.arguments(posonlyargs=[], args=[], kwonlyargs=[], kw_defaults=[], defaults=[]), body=v)
                for v in node.values]
        return ast.copy_location(ast.Call(func=ast.Attribute(value=ast.Name(id="_jst", ctx=ast.Load()), attr=fn, ctx=ast.Load()),
                                          args=args, keywords=[]), node)

    def visit_UnaryOp(self, node):
        self.generic_visit(node)
        if isinstance(node.op, ast.Not):
            return ast.copy_location(ast.Call(func=ast.Attribute(value=ast.Name(id="_jst", ctx=ast.Load()), attr="not_", ctx=ast.Load()),
                                              args=[node.operand], keywords=[]), node)
        return node

    def visit_If(self, node):
        self.generic_visit(node)
        if _has_jump(node.body) or _has_jump(node.orelse):
            return node
        names = _assigned_names(node.body + node.orelse)
        if not names:
            return node
        uid = self._uid()
        nl = f"nonlocal {', '.join(names)}"

        def fn(name, body):
            f = _parse_stmt(f"def {name}():\n    {nl}\n    pass")[0]
            f.body = [f.body[0]] + (body or [ast.Pass()])
            return f
        call = _parse_stmt(
            f"({', '.join(names)}{',' if len(names) == 1 else ''}) = _jst.convert_ifelse(__jst_pred_{uid}, __jst_true_{uid}, "
            f"__jst_false_{uid}, __jst_get_{uid}, __jst_set_{uid}, {names!r})")[0]
        pred = ast.Assign(targets=[ast.Name(id=f"__jst_pred_{uid}", ctx=ast.Store())], value=node.test)
        out = self._prelude(names) + [pred, fn(f"__jst_true_{uid}", node.body), fn(f"__jst_false_{uid}", node.orelse)] \
            + self._accessors(uid, names) + [call]
        return [ast.copy_location(n, node) for n in out]

    def visit_For(self, node):
        """``for i in range(...)`` becomes a counted ``while`` (so that a tensor bound gives a graph loop)."""
        it = node.iter
        if not (isinstance(it, ast.Call) and isinstance(it.func, ast.Name) and it.func.id == "range" and not it.keywords
                and 1 <= len(it.args) <= 3 and isinstance(node.target, ast.Name) and not node.orelse
                and not _has_jump(node.body)):
            self.generic_visit(node)
            return node
        uid = self._uid()
        a = it.args
        start = a[0] if len(a) >= 2 else ast.Constant(value=0)
        stop = a[1] if len(a) >= 2 else a[0]
        step = a[2] if len(a) == 3 else ast.Constant(value=1)
        c, e, st = f"__jst_i_{uid}", f"__jst_stop_{uid}", f"__jst_step_{uid}"
        init = [ast.Assign(targets=[ast.Name(id=c, ctx=ast.Store())], value=start),
                ast.Assign(targets=[ast.Name(id=e, ctx=ast.Store())], value=stop),
                ast.Assign(targets=[ast.Name(id=st, ctx=ast.Store())], value=step)]
        loop = _parse_stmt(f"while _jst.range_cond({c}, {e}, {st}):\n    {node.target.id} = {c}\n    {c} = {c} + {st}")[0]
        loop.body = [loop.body[0]] + node.body + [loop.body[1]]
        out = init + [loop]
        out = [ast.copy_location(n, node) for n in out]
        for n in out:
            ast.fix_missing_locations(n)
        res = []
        for n in out:
            r = self.visit(n)
            res.extend(r if isinstance(r, list) else [r])
        return res

    def visit_While(self, node):
        self.generic_visit(node)
        if _has_jump(node.body) or node.orelse:
            return node
        names = _assigned_names(node.body)
        if not names:
            return node
        uid = self._uid()
        nl = f"nonlocal {', '.join(names)}"
        cond = _parse_stmt(f"def __jst_cond_{uid}():\n    return None")[0]
        cond.body = [ast.Return(value=node.test)]
        body = _parse_stmt(f"def __jst_body_{uid}():\n    {nl}\n    pass")[0]
        body.body = [body.body[0]] + node.body
        call = _parse_stmt(
            f"({', '.join(names)}{',' if len(names) == 1 else ''}) = _jst.convert_while(__jst_cond_{uid}, __jst_body_{uid}, "
            f"__jst_get_{uid}, __jst_set_{uid}, {names!r})")[0]
        out = self._prelude(names) + [cond, body] + self._accessors(uid, names) + [call]
        return [ast.copy_location(n, node) for n in out]


def _lift_early_returns(stmts):
    """``if c: ...; return X`` followed by more statements becomes ``if c: ...; __jst_ret = X`` / ``else: <rest>`` with
    one ``return __jst_ret`` at the end, so that the ``if`` has no jump and can be converted (the reference's
    ReturnTransformer handles the general case; this covers a return as the LAST statement of a branch)."""
    def ends_with_return(body):
        return bool(body) and isinstance(body[-1], ast.Return)

    def only_tail_return(body):
        return ends_with_return(body) and not _has_jump(body[:-1])

    def to_assign(ret):
        return ast.Assign(targets=[ast.Name(id="__jst_ret", ctx=ast.Store())],
                          value=ret.value if ret.value is not None else ast.Constant(value=None))

    def lift(body):
        """Returns a statement list without returns that leaves the result in ``__jst_ret``, or None."""
        for i, st in enumerate(body):
            if isinstance(st, ast.Return):
                return body[:i] + [to_assign(st)] if not _has_jump(body[:i]) else None
            if isinstance(st, ast.If) and (_has_jump(st.body) or _has_jump(st.orelse)):
                if _has_jump(body[:i]):
                    return None
                rest = body[i + 1:]
                t = lift(st.body) if ends_with_return(st.body) or _has_jump(st.body) else st.body
                if t is None:
                    return None
                if ends_with_return(st.body) or _returns_on_all_paths(st.body):
                    f = lift(st.orelse + rest)
                else:
                    return None
                if f is None:
                    return None
                new_if = ast.If(test=st.test, body=t, orelse=f)
                return body[:i] + [ast.copy_location(new_if, st)]
            if _has_jump([st]):
                return None
        return body + [ast.Assign(targets=[ast.Name(id="__jst_ret", ctx=ast.Store())], value=ast.Constant(value=None))]

    if not any(isinstance(st, ast.If) and _has_jump(st.body + st.orelse) for st in stmts):
        return stmts
    lifted = lift(stmts)
    if lifted is None:
        return stmts
    return lifted + [ast.Return(value=ast.Name(id="__jst_ret", ctx=ast.Load()))]


def _returns_on_all_paths(body):
    if not body:
        return False
    last = body[-1]
    if isinstance(last, ast.Return):
        return True
    if isinstance(last, ast.If):
        return _returns_on_all_paths(last.body) and _returns_on_all_paths(last.orelse)
    return False


_converted = {}


def convert_function(fn):
    """Returns ``fn`` with tensor-capable control flow (or ``fn`` itself when its source is not available)."""
    raw = getattr(fn, "__func__", fn)
    if raw in _converted:
        new = _converted[raw]
    else:
        try:
            src = textwrap.dedent(inspect.getsource(raw))
            tree = ast.parse(src)
        except (OSError, TypeError, SyntaxError, IndentationError):
            return fn
        fdef = tree.body[0]
        if not isinstance(fdef, (ast.FunctionDef, ast.AsyncFunctionDef)):
            return fn
        fdef.decorator_list = []
        fdef.body = _lift_early_returns(fdef.body)
        ast.fix_missing_locations(tree)
        _Transformer().visit(fdef)
        ast.fix_missing_locations(tree)
        import sys
        from . import dy2static as _self
        glb = dict(raw.__globals__)
        glb["_jst"] = _self
        # free variables of the original become globals of the converted copy (values at conversion time)
        if raw.__closure__:
            for name, cell in zip(raw.__code__.co_freevars, raw.__closure__):
                try:
                    glb[name] = cell.cell_contents
                except ValueError:
                    pass
        loc = {}
        try:
            exec(compile(tree, filename=f"<dy2static {raw.__name__}>", mode="exec"), glb, loc)
        except SyntaxError:
            return fn
        new = functools.wraps(raw)(loc[fdef.name])
        _converted[raw] = new
    if hasattr(fn, "__self__"):
        return new.__get__(fn.__self__, type(fn.__self__))
    return new


# ----------------------------------------------------------------------------------------- program-backed callable
class ProgramFunction:
    """``to_static(full_graph=True)``: one recorded ``static.Program`` per input signature."""

    def __init__(self, fn, layer=None):
        self._orig = fn
        self._fn = convert_function(fn)
        self._layer = layer
        self._programs = {}

    def _signature(self, tensors, consts):
        training = getattr(self._layer, "training", None)
        return (tuple((tuple(t.shape), t.dtype) for t in tensors), consts, training)

    def concrete_program(self, *args):
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        consts = tuple(a for a in args if not isinstance(a, torch.Tensor))
        return self._programs.get(self._signature(tensors, consts))

    def __call__(self, *args):
        from .. import static
        from ..static import graph as g
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        consts = tuple(a if isinstance(a, (int, float, str, bool, type(None))) else id(a)
                       for a in args if not isinstance(a, torch.Tensor))
        key = self._signature(tensors, consts)
        ent = self._programs.get(key)
        if ent is None:
            was_static = g._S.enabled
            prog = static.Program()
            if not was_static:
                g.enable()
            try:
                with static.program_guard(prog, static.Program()):
                    holders, it = [], iter(range(len(tensors)))
                    call_args = []
                    for a in args:
                        if isinstance(a, torch.Tensor):
                            i = next(it)
                            h = static.data(f"arg{i}", list(a.shape), a.dtype)
                            with g.suspend():
                                h.as_subclass(torch.Tensor).copy_(a.detach().as_subclass(torch.Tensor))
                                h.stop_gradient = not a.requires_grad
                            holders.append(h)
                            call_args.append(h)
                        else:
                            call_args.append(a)
                    out = self._fn(*call_args)
            finally:
                if not was_static:
                    g.disable()
            flat, spec = torch.utils._pytree.tree_flatten(out)
            fetch = [o for o in flat if isinstance(o, torch.Tensor)]
            prog._nodes[:] = g.prune(prog._nodes, [prog._slot_of(o) for o in fetch]) if fetch else prog._nodes
            ent = self._programs[key] = (prog, [h.name for h in holders], flat, spec, fetch)
        prog, names, flat, spec, fetch = ent
        prog._needs_grad = torch.is_grad_enabled()
        env_feed = dict(zip(names, tensors))
        with g.suspend():
            outs = prog._execute(env_feed, fetch, keep_graph=True)
        it = iter(outs)
        res = [as_tensor(next(it)) if isinstance(o, torch.Tensor) else o for o in flat]
        return torch.utils._pytree.tree_unflatten(res, spec)
