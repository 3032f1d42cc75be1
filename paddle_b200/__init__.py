"""paddle_b200 — a Blackwell-native deep-learning framework with PaddlePaddle's Python API.

PyTorch supplies the tensor storage, dispatcher and autograd engine; the hot operators are
hand-written sm_100a CUDA kernels (``paddle_b200/csrc/kernels``), the distributed layer is one process
per GPU over NCCL plus fused compute+collective kernels on symmetric memory.  ``import paddle``
resolves to this package through the alias package at the repository root.
"""
from __future__ import annotations

import torch as _torch

__version__ = "0.1.0"
full_version = __version__
commit = "b200-native"

from ._core import dtype as _dt  # noqa: E402
from ._core import unique_name  # noqa: E402,F401
from ._core.dtype import (CPUPlace, CUDAPinnedPlace, CUDAPlace, get_default_dtype, get_device,  # noqa: E402,F401
                          set_default_dtype, set_device)
from ._core.tensor import EagerParamBase, Parameter, Tensor, as_tensor, to_tensor  # noqa: E402,F401

# dtypes are the torch dtype objects
float32 = _torch.float32
float64 = _torch.float64
float16 = _torch.float16
bfloat16 = _torch.bfloat16
int8 = _torch.int8
uint8 = _torch.uint8
int16 = _torch.int16
int32 = _torch.int32
int64 = _torch.int64
bool = _torch.bool  # noqa: A001
complex64 = _torch.complex64
complex128 = _torch.complex128
float8_e4m3fn = _torch.float8_e4m3fn
float8_e5m2 = _torch.float8_e5m2
dtype = _torch.dtype

from .tensor import *  # noqa: E402,F401,F403
from .tensor import creation, linalg, manipulation, math, random  # noqa: E402,F401
from .tensor.random import seed  # noqa: E402,F401
from . import tensor  # noqa: E402,F401

from .autograd import enable_grad, grad, is_grad_enabled, no_grad, set_grad_enabled  # noqa: E402,F401
from . import autograd  # noqa: E402,F401
from . import nn  # noqa: E402,F401
from .nn.layer.layers import ParamAttr  # noqa: E402,F401
from . import optimizer  # noqa: E402,F401
from . import amp  # noqa: E402,F401
from . import framework  # noqa: E402,F401
from .framework import async_save, get_flags, load, save, set_flags  # noqa: E402,F401
from .framework.random import get_cuda_rng_state, get_rng_state, set_cuda_rng_state, set_rng_state  # noqa: E402,F401
from .ops.functional import get_kernel_policy, set_kernel_policy  # noqa: E402,F401


def _bind_tensor_methods():
    """Expose the functional API as Tensor methods (the reference does this in
    python/paddle/base/dygraph/math_op_patch.py and tensor_patch_methods.py)."""
    import types

    from .tensor import linalg as _l
    from .tensor import manipulation as _mp
    from .tensor import math as _m
    skip = set(dir(Tensor)) - set(dir(_torch.Tensor))  # keep explicit overrides in the subclass
    taken = set()
    for mod in (_m, _mp, _l):
        for name, fn in vars(mod).items():
            if name.startswith("_") or not isinstance(fn, types.FunctionType) or fn.__module__ != mod.__name__:
                continue
            if name in skip or name in taken:
                continue
            if hasattr(_torch.Tensor, name) and name not in _PADDLE_SEMANTIC_METHODS:
                continue  # same-named torch method keeps torch semantics unless listed
            setattr(Tensor, name, fn)
            taken.add(name)
    for name in ("add", "subtract", "multiply", "divide"):
        inplace = name + "_"
        if not hasattr(Tensor, inplace):
            tfn = {"add": "add_", "subtract": "sub_", "multiply": "mul_", "divide": "div_"}[name]
            setattr(Tensor, inplace, (lambda t: lambda self, y, name=None: getattr(_torch.Tensor, t)(self, y))(tfn))


_PADDLE_SEMANTIC_METHODS = {
    "roll", "flip", "cast", "index_select", "masked_select", "nonzero", "sort", "argsort", "unique", "kthvalue",
    "mode", "median", "logsumexp", "cumprod", "take_along_axis", "put_along_axis", "scatter", "scatter_",
    "index_add", "repeat_interleave", "moveaxis", "diff", "count_nonzero", "clip", "pow", "equal", "where",
    "slice", "stack", "expand_as", "broadcast_to", "logical_and", "logical_or", "logical_not", "logical_xor",
    "quantile", "trace", "diagonal", "cross", "dot", "dist", "tensordot", "allclose", "isclose", "equal_all",
    "bmm", "mm", "mv", "inverse", "cholesky", "floor_divide", "remainder", "maximum", "minimum", "lerp",
    "nan_to_num", "masked_fill", "tril", "triu",
}
_bind_tensor_methods()
Tensor.clip = math.clip
Tensor.tril = lambda self, diagonal=0: _torch.tril(self, diagonal)
Tensor.triu = lambda self, diagonal=0: _torch.triu(self, diagonal)


from .tensor import extras as _extras  # noqa: E402
for _n, _v in vars(_extras).items():
    if not _n.startswith("_") and _n not in globals():
        globals()[_n] = _v
for _n, _v in _extras._make_inplace_table().items():
    if _n not in globals():
        globals()[_n] = _v
    if not hasattr(Tensor, _n):
        setattr(Tensor, _n, _v)
del _n, _v
# remaining Tensor methods of the reference's tensor_method_func list that exist as functions
import importlib as _il  # noqa: E402
_la = _il.import_module(__name__ + ".linalg")
for _n in ("create_parameter", "histogram_bin_edges", "matrix_transpose", "reduce_as", "multigammaln", "block_diag", "isin",
           "gammaincc", "gammainc", "reverse", "gammaln", "bitwise_invert", "cumulative_trapezoid", "polar", "i0e", "i1",
           "i1e", "combinations", "top_p_sampling", "put_along_axis_", "pca_lowrank", "svd_lowrank", "create_tensor"):
    _v = globals().get(_n) or getattr(_la, _n, None)
    if _v is None and _n == "create_tensor":
        _v = lambda self, dtype=None, name=None, persistable=False: zeros([0], dtype or self.dtype)   # noqa: E731
    if _v is not None and not hasattr(Tensor, _n):
        setattr(Tensor, _n, _v)
del _n, _v

from .tensor import semantics as _semantics  # noqa: E402
_semantics.install(globals())


def is_compiled_with_ipu():
    return False


def is_compiled_with_cuda():
    return True


def is_compiled_with_rocm():
    return False


def is_compiled_with_xpu():
    return False


def is_compiled_with_cinn():
    return False


def is_compiled_with_custom_device(name=None):
    return False


def in_dynamic_mode():
    from .static import graph as _sg
    return not _sg._S.enabled


in_dygraph_mode = in_dynamic_mode


def enable_static():
    """Static-graph mode: calls are recorded into the current ``static.Program`` and replayed by ``static.Executor``."""
    from .static import graph as _sg
    _sg.enable()


def disable_static(place=None):
    from .static import graph as _sg
    _sg.disable()
    if place is not None:
        set_device(place)


def disable_signal_handler():
    pass


def summary(net, input_size=None, dtypes=None, input=None):
    from .hapi import summary as _s
    return _s(net, input_size, dtypes, input)


def flops(net, input_size, custom_ops=None, print_detail=False):
    from .hapi import flops as _f
    return _f(net, input_size, custom_ops, print_detail)


def check_shape(shape):
    return shape


def get_cudnn_version():
    return _torch.backends.cudnn.version()


def set_printoptions(precision=None, threshold=None, edgeitems=None, sci_mode=None, linewidth=None):
    from .tensor.to_string import set_printoptions as _set
    _set(precision, threshold, edgeitems, sci_mode, linewidth)


def set_grad_enabled_ctx(mode):
    return _torch.set_grad_enabled(mode)


_lazy_depth = [0]


def _lazy_init_active():
    return _lazy_depth[0] > 0


class LazyGuard:
    """Layers built inside the guard get parameters whose initial values are not computed until
    ``param.initialize()`` is called (python/paddle/nn/initializer/lazy_init.py)."""

    def __enter__(self):
        _lazy_depth[0] += 1
        return self

    def __exit__(self, *a):
        _lazy_depth[0] -= 1
        return False


_LAZY_SUBMODULES = {
    "distributed", "io", "device", "jit", "static", "profiler", "incubate", "vision", "text", "audio", "metric",
    "hapi", "distribution", "sparse", "fft", "signal", "quantization", "geometric", "utils", "inference",
    "models", "parallel", "regularizer", "callbacks", "hub", "onnx", "sysconfig", "version", "base", "reader",
    "dataset", "_C_ops", "_legacy_C_ops", "cuda", "decomposition", "tensorrt", "cost_model",
}


# flags given as FLAGS_<name> environment variables act like set_flags at import
from .framework import flags as _flags_mod  # noqa: E402
_flags_mod._apply_env_effects()

def __getattr__(name):
    if name in _LAZY_SUBMODULES:
        import importlib
        try:
            mod = importlib.import_module(f"{__name__}.{name}")
        except ModuleNotFoundError as e:
            if e.name == f"{__name__}.{name}":
                raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
            raise
        globals()[name] = mod
        return mod
    if name == "Model":
        from .hapi import Model
        return Model
    if name == "DataParallel":
        from .distributed.parallel import DataParallel
        return DataParallel
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
