"""``paddle.utils.cpp_extension`` (python/paddle/utils/cpp_extension/cpp_extension.py:79-950, extension_utils.py):
build out-of-tree C++ / CUDA operators written against ``paddle/extension.h`` and expose every ``PD_BUILD_OP`` as a
Python function, with autograd wired to its ``PD_BUILD_GRAD_OP``.

``load(name, sources)`` compiles just in time (ninja; CUDA sources for sm_100a only) and returns a module whose
attributes are the operators.  ``setup(name=..., ext_modules=CUDAExtension(sources))`` builds and installs the same
thing ahead of time; the installed package imports through ``load_op_module``.  The header shipped under
``paddle_b200/include`` implements the reference's extension API over ATen, so a custom kernel sees the framework's
device memory, current stream and allocator."""
from __future__ import annotations

import os
import types

import torch
import torch.utils.cpp_extension as _t

SM100_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"]
_BIND_SRC = """// generated: exposes the custom-operator registry of this shared object
#include "paddle/extension.h"
PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) { paddle::bind_ops(m); }
"""


def get_include():
    """Directory holding ``paddle/extension.h``."""
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")


def get_build_directory(verbose=False):
    """``$PADDLE_EXTENSION_DIR`` or torch's extension cache."""
    root = os.environ.get("PADDLE_EXTENSION_DIR")
    if root:
        os.makedirs(root, exist_ok=True)
        return root
    return _t._get_build_directory("", verbose)


def _slot(name):
    """``X@GRAD`` / ``X@VECTOR`` / ``X@OPTIONAL`` -> (base name, is grad, is list, is optional)."""
    base, grad, vec, opt = name, False, False, False
    changed = True
    while changed:
        changed = False
        for suffix in ("@GRAD", "@VECTOR", "@OPTIONAL"):
            if base.endswith(suffix):
                base = base[:-len(suffix)]
                grad, vec, opt = grad or suffix == "@GRAD", vec or suffix == "@VECTOR", opt or suffix == "@OPTIONAL"
                changed = True
    return base, grad, vec, opt


def _attr_names(attrs):
    return [a.split(":")[0].strip() for a in attrs]


_ATTR_CAST = {"bool": bool, "int": int, "float": float, "int64_t": int, "std::string": str,
              "std::vector<int>": lambda v: [int(x) for x in v], "std::vector<float>": lambda v: [float(x) for x in v],
              "std::vector<int64_t>": lambda v: [int(x) for x in v], "std::vector<std::string>": lambda v: [str(x) for x in v]}


def _cast_attr(decl, value):
    typ = decl.split(":", 1)[1].strip() if ":" in decl else ""
    fn = _ATTR_CAST.get(typ)
    return fn(value) if fn is not None else value


def _wrap_out(t):
    from .._core.tensor import as_tensor
    if isinstance(t, (list, tuple)):
        return [_wrap_out(x) for x in t]
    return as_tensor(t) if isinstance(t, torch.Tensor) else t


def _make_op(ext, name, metas):
    meta = metas[name]
    grad_meta = metas.get(name + "_grad")
    in_slots = [_slot(n) for n in meta["inputs"]]
    out_names = [_slot(n)[0] for n in meta["outputs"]]
    attr_decls = list(meta["attrs"])
    attr_names = _attr_names(attr_decls)

    def raw_forward(inputs, attrs):
        return list(ext.run(name, list(inputs) + list(attrs)))

    def split_call(args, kwargs):
        args = list(args)
        n_in = len(in_slots)
        inputs = args[:n_in]
        rest = args[n_in:]
        for (base, _, _, opt) in in_slots[len(inputs):]:
            if base in kwargs:
                inputs.append(kwargs.pop(base))
            elif base.lower() in kwargs:
                inputs.append(kwargs.pop(base.lower()))
            elif opt:
                inputs.append(None)
            else:
                raise TypeError(f"{name}() missing input {base!r}")
        attrs = []
        for i, (decl, an) in enumerate(zip(attr_decls, attr_names)):
            if i < len(rest):
                attrs.append(_cast_attr(decl, rest[i]))
            elif an in kwargs:
                attrs.append(_cast_attr(decl, kwargs.pop(an)))
            else:
                raise TypeError(f"{name}() missing attribute {an!r}")
        if kwargs:
            raise TypeError(f"{name}() got unexpected arguments {sorted(kwargs)}")
        return inputs, attrs

    if grad_meta is None:
        def op(*args, **kwargs):
            inputs, attrs = split_call(args, kwargs)
            outs = _wrap_out(raw_forward(inputs, attrs))
            return outs[0] if len(outs) == 1 else tuple(outs)
    else:
        g_in = [_slot(n) for n in grad_meta["inputs"]]
        g_out = [_slot(n) for n in grad_meta["outputs"]]
        g_attr_names = _attr_names(grad_meta["attrs"])
        in_index = {s[0]: i for i, s in enumerate(in_slots)}
        out_index = {n: i for i, n in enumerate(out_names)}
        for base, is_grad, _, _ in g_out:
            if not is_grad or base not in in_index:
                raise ValueError(f"grad operator of {name}: output {base!r} must be paddle::Grad of a forward input")

        class _Fn(torch.autograd.Function):
            @staticmethod
            def forward(ctx, attrs, layout, out_box, *flat):
                # flat: the forward inputs with list slots flattened; layout: per slot None (tensor), -1 (absent) or a length
                inputs, pos = [], 0
                for n in layout:
                    if n is None:
                        inputs.append(flat[pos])
                        pos += 1
                    elif n == -1:
                        inputs.append(None)
                    else:
                        inputs.append(list(flat[pos:pos + n]))
                        pos += n
                outs = raw_forward(inputs, attrs)
                ctx.attrs, ctx.layout = attrs, layout
                ctx.n_flat = len(flat)
                saved, plan = [], []
                for base, is_grad, vec, _ in g_in:
                    if is_grad:
                        plan.append(("grad", out_index[base]))
                        continue
                    src = inputs[in_index[base]] if base in in_index else outs[out_index[base]]
                    if isinstance(src, (list, tuple)):
                        plan.append(("list", len(saved), len(src)))
                        saved += list(src)
                    elif src is None:
                        plan.append(("none",))
                    else:
                        plan.append(("one", len(saved)))
                        saved.append(src)
                ctx.plan = plan
                ctx.save_for_backward(*saved)
                flat_out = []
                ctx.out_layout = []
                for o in outs:
                    if isinstance(o, (list, tuple)):
                        ctx.out_layout.append(len(o))
                        flat_out += list(o)
                    else:
                        ctx.out_layout.append(None)
                        flat_out.append(o)
                out_box.extend(ctx.out_layout)
                return tuple(flat_out)

            @staticmethod
            def backward(ctx, *gflat):
                saved = ctx.saved_tensors
                gouts, pos = [], 0
                for n in ctx.out_layout:
                    if n is None:
                        gouts.append(gflat[pos])
                        pos += 1
                    else:
                        gouts.append(list(gflat[pos:pos + n]))
                        pos += n
                args = []
                for p in ctx.plan:
                    if p[0] == "grad":
                        g = gouts[p[1]]
                        args.append(g.contiguous() if isinstance(g, torch.Tensor) else g)
                    elif p[0] == "one":
                        args.append(saved[p[1]])
                    elif p[0] == "list":
                        args.append(list(saved[p[1]:p[1] + p[2]]))
                    else:
                        args.append(None)
                fwd_attr = dict(zip(attr_names, ctx.attrs))
                args += [fwd_attr[a] for a in g_attr_names]
                gins = list(ext.run(name + "_grad", args))
                by_input = {}
                for (base, _, _, _), g in zip(g_out, gins):
                    by_input[in_index[base]] = g
                grads = []
                for i, n in enumerate(ctx.layout):
                    g = by_input.get(i)
                    if n is None:
                        grads.append(g)
                    elif n == -1:
                        continue
                    else:
                        grads += list(g) if g is not None else [None] * n
                return (None, None, None, *grads)

        def op(*args, **kwargs):
            inputs, attrs = split_call(args, kwargs)
            layout, flat = [], []
            for v in inputs:
                if v is None:
                    layout.append(-1)
                elif isinstance(v, (list, tuple)):
                    layout.append(len(v))
                    flat += list(v)
                else:
                    layout.append(None)
                    flat.append(v)
            out_box = []
            flat_out = list(_Fn.apply(attrs, tuple(layout), out_box, *flat))
            outs, pos = [], 0
            for n in out_box:
                if n is None:
                    outs.append(flat_out[pos])
                    pos += 1
                else:
                    outs.append(flat_out[pos:pos + n])
                    pos += n
            outs = _wrap_out(outs)
            return outs[0] if len(outs) == 1 else tuple(outs)

    op.__name__ = name
    op.__doc__ = (f"custom operator {name}({', '.join([s[0] for s in in_slots] + attr_names)}) -> {', '.join(out_names)}"
                  + ("; differentiable" if grad_meta is not None else ""))
    op.meta = meta
    return op


def load_op_module(ext, name=None):
    """Python module with one function per operator registered in the built extension ``ext``."""
    names = list(ext.op_names())
    metas = {n: dict(ext.op_meta(n)) for n in names}
    mod = types.ModuleType(name or getattr(ext, "__name__", "custom_ops"))
    mod.__ext__ = ext
    for n in names:
        if n.endswith("_grad") and n[:-5] in metas or n.endswith("_grad_grad"):
            continue
        setattr(mod, n, _make_op(ext, n, metas))
    mod.__all__ = [n for n in names if hasattr(mod, n)]

    def infer_shape(op_name, *shapes_and_attrs):
        return [list(s) for s in ext.infer_shape(op_name, list(shapes_and_attrs))]

    def infer_dtype(op_name, *dtypes):
        return list(ext.infer_dtype(op_name, list(dtypes)))
    mod.infer_shape, mod.infer_dtype = infer_shape, infer_dtype
    return mod


def _with_binding(name, sources, build_directory):
    bind = os.path.join(build_directory, f"{name}_pd_bind.cc")
    if not os.path.exists(bind) or open(bind).read() != _BIND_SRC:
        with open(bind, "w") as f:
            f.write(_BIND_SRC)
    return list(sources) + [bind]


def load(name, sources, extra_cxx_cflags=None, extra_cuda_cflags=None, extra_ldflags=None, extra_include_paths=None,
         extra_library_paths=None, build_directory=None, verbose=False, **kw):
    """Compile ``sources`` (``.cc`` / ``.cpp`` with the host compiler, ``.cu`` with nvcc for sm_100a) and return the
    operator module.  Rebuilds only when a source or a flag changed."""
    build_directory = build_directory or os.path.join(get_build_directory(verbose), name)
    os.makedirs(build_directory, exist_ok=True)
    ldflags = list(extra_ldflags or []) + [f"-L{p}" for p in (extra_library_paths or [])]
    has_cuda = any(str(s).endswith((".cu", ".cuh")) for s in sources)
    ext = _t.load(name=name, sources=_with_binding(name, sources, build_directory), extra_cflags=list(extra_cxx_cflags or []),
                  extra_cuda_cflags=(list(extra_cuda_cflags or []) + SM100_FLAGS) if has_cuda else None, extra_ldflags=ldflags,
                  extra_include_paths=[get_include()] + list(extra_include_paths or []), build_directory=build_directory,
                  verbose=verbose, with_cuda=has_cuda or None)
    return load_op_module(ext, name)


def _extension(factory, sources, args, kwargs, cuda):
    name = kwargs.pop("name", None) or "custom_ops"
    inc = list(kwargs.pop("include_dirs", [])) + [get_include()]
    if cuda:
        eca = kwargs.setdefault("extra_compile_args", {})
        if isinstance(eca, dict):
            eca["nvcc"] = list(eca.get("nvcc", [])) + SM100_FLAGS
    build_tmp = os.path.join(os.getcwd(), "build")
    os.makedirs(build_tmp, exist_ok=True)
    return factory(name, _with_binding(name, sources, build_tmp), *args, include_dirs=inc, **kwargs)


def CppExtension(sources, *args, **kwargs):
    return _extension(_t.CppExtension, sources, args, kwargs, cuda=False)


def CUDAExtension(sources, *args, **kwargs):
    return _extension(_t.CUDAExtension, sources, args, kwargs, cuda=True)


BuildExtension = _t.BuildExtension


def setup(**attr):
    """``setuptools.setup`` with the extension builder preset; ``ext_modules`` may be a single extension.  A stub
    ``<name>.py`` importing the built library through ``load_op_module`` is added as ``py_modules``."""
    from setuptools import setup as _setup
    ext = attr.get("ext_modules")
    if ext is not None and not isinstance(ext, (list, tuple)):
        attr["ext_modules"] = [ext]
    if attr.get("ext_modules") and "name" not in attr:
        attr["name"] = attr["ext_modules"][0].name
    attr.setdefault("cmdclass", {"build_ext": BuildExtension.with_options(no_python_abi_suffix=True)})
    return _setup(**attr)
