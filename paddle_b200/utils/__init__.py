"""``paddle.utils``"""
from __future__ import annotations

import functools
import warnings

from . import cpp_extension, dlpack, download, unique_name  # noqa: F401


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


def require_version(min_version, max_version=None):
    """Raises if the installed framework version is outside ``[min_version, max_version]``
    (python/paddle/utils/__init__.py ``require_version``; a development build, version 0.0.0, always passes)."""
    from ..version import full_version
    if not isinstance(min_version, str) or (max_version is not None and not isinstance(max_version, str)):
        raise TypeError("The type of 'min_version' / 'max_version' in require_version must be str")

    def parse(v):
        parts = [int(x) for x in v.split(".")[:4] if x.isdigit()]
        if not parts:
            raise ValueError(f"The value of version in require_version must be in format '\\d+(\\.\\d+){{0,3}}', but received {v}")
        return parts + [0] * (4 - len(parts))
    lo = parse(min_version)
    hi = parse(max_version) if max_version is not None else None
    cur = parse(full_version.split("+")[0]) if full_version[0].isdigit() else [0, 0, 0, 0]
    if cur == [0, 0, 0, 0]:
        return
    if cur < lo or (hi is not None and cur > hi):
        raise Exception(f"VersionError: the installed version {full_version} does not satisfy "
                        f"[{min_version}, {max_version or 'inf'}]")
