"""``paddle.base``: the legacy namespace that static-graph scripts import their building blocks from
(python/paddle/base/__init__.py)."""
from ..static import (BuildStrategy, CompiledProgram, Executor, Program, Variable, default_main_program,  # noqa: F401
                      default_startup_program, global_scope, name_scope, program_guard, scope_guard)
from ..static import graph as framework  # noqa: F401
from ..nn.layer.layers import ParamAttr  # noqa: F401
from .. import CPUPlace, CUDAPlace  # noqa: F401

__all__ = []


def in_dygraph_mode():
    from .. import in_dynamic_mode
    return in_dynamic_mode()


def is_compiled_with_cuda():
    import torch
    return torch.cuda.is_available()


class _Core:
    """``paddle.base.core``: the names scripts take from the reference's binding module that make sense here."""
    from ..framework.errors import EnforceNotMet  # noqa: F401

    class EOFException(Exception):
        """Raised by readers at the end of data (paddle.base.core.EOFException)."""

    @staticmethod
    def is_compiled_with_cuda():
        return is_compiled_with_cuda()

    @staticmethod
    def get_cuda_device_count():
        import torch
        return torch.cuda.device_count()


core = _Core()
