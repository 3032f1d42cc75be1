"""``paddle.utils.cpp_extension``: JIT-build custom C++/CUDA operators
(python/paddle/utils/cpp_extension/cpp_extension.py) on torch.utils.cpp_extension; CUDA sources are compiled
for sm_100a only."""
from __future__ import annotations

import torch.utils.cpp_extension as _t

SM100_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"]


def load(name, sources, extra_cxx_cflags=None, extra_cuda_cflags=None, extra_ldflags=None, extra_include_paths=None,
         build_directory=None, verbose=False, **kw):
    return _t.load(name=name, sources=sources, extra_cflags=extra_cxx_cflags,
                   extra_cuda_cflags=(extra_cuda_cflags or []) + SM100_FLAGS, extra_ldflags=extra_ldflags,
                   extra_include_paths=extra_include_paths, build_directory=build_directory, verbose=verbose)


def CppExtension(sources, *args, **kwargs):
    return _t.CppExtension(kwargs.pop("name", "custom_ops"), sources, *args, **kwargs)


def CUDAExtension(sources, *args, **kwargs):
    kwargs.setdefault("extra_compile_args", {"nvcc": SM100_FLAGS})
    return _t.CUDAExtension(kwargs.pop("name", "custom_ops"), sources, *args, **kwargs)


BuildExtension = _t.BuildExtension


def setup(**attr):
    from setuptools import setup as _setup
    attr.setdefault("cmdclass", {"build_ext": BuildExtension})
    return _setup(**attr)


def get_build_directory():
    return _t._get_build_directory("", False)
