"""Legacy operator names still referenced from Python (``_legacy_C_ops.c_identity`` ...)."""
from ._C_ops import __getattr__  # noqa: F401
