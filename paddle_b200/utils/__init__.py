"""``paddle.utils``"""
from __future__ import annotations

import functools
import warnings

from .._core import unique_name  # noqa: F401
from . import cpp_extension, dlpack  # noqa: F401


def deprecated(update_to="", since="", reason="", level=0):
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **k):
            warnings.warn(f"{fn.__name__} is deprecated since {since}: {reason} {update_to}", DeprecationWarning)
            return fn(*a, **k)
        return wrapper
    return deco


def try_import(name):
    import importlib
    return importlib.import_module(name)


def run_check():
    """``paddle.utils.run_check``: one tiny training step on every visible device."""
    import torch

    import paddle_b200 as paddle
    n = torch.cuda.device_count()
    l = paddle.nn.Linear(4, 4)
    x = paddle.randn([2, 4])
    l(x).sum().backward()
    print(f"paddle_b200 works on {'%d GPU(s)' % n if n else 'CPU'}; native kernels: "
          f"{'available' if n else 'not loaded (no GPU)'}")
    return True


def flatten(nest):
    out = []
    for n in (nest if isinstance(nest, (list, tuple)) else [nest]):
        out.extend(flatten(n) if isinstance(n, (list, tuple)) else [n])
    return out
