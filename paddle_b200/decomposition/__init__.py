"""Operator decomposition (python/paddle/decomposition/__init__.py): composite operators of a recorded program are
rewritten into a closed set of primitive operators, so that passes and back ends after it only have to know those.

The reference keeps most rules in C++ (paddle/fluid/primitive/composite/composite.h) and applies them to PIR programs;
here a rule is a Python function over the primitive operators of :mod:`.primitives`, and :func:`decompose` re-traces it
into the recorded program in place of the composite node."""
from . import rules  # noqa: F401
from .decomp import decompose, is_primitive_program  # noqa: F401
from .primitives import PRIMITIVES  # noqa: F401
from .register import get_decomp_rule, register_decomp, registered_ops  # noqa: F401
