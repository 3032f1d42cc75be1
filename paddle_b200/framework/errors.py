"""Typed errors (paddle/common/errors.h:28-147 error codes; paddle/fluid/pybind/exception.cc:39-80 maps them onto
Python's built-in exception classes).  ``EnforceNotMet`` is the common base, as ``paddle.base.core.EnforceNotMet``; every
typed error also derives from the built-in class the reference raises for its code, so ``except ValueError`` around an
invalid-argument failure behaves as it does with the reference."""
from __future__ import annotations


class EnforceNotMet(Exception):
    """Base of every error the framework raises on a failed check."""
    code = 0
    type_string = "Error"

    def __init__(self, message="", *args):
        super().__init__(message, *args)
        self.message = str(message)

    def __str__(self):
        return f"({self.type_string}) {self.message}" if self.message else self.type_string


def _typed(name, code, type_string, builtin):
    cls = type(name, (EnforceNotMet, builtin), {"code": code, "type_string": type_string, "__doc__":
               f"Error code {code} ({type_string}); also a ``{builtin.__name__}``."})
    cls.__module__ = __name__
    return cls


InvalidArgumentError = _typed("InvalidArgumentError", 1, "InvalidArgumentError", ValueError)
NotFoundError = _typed("NotFoundError", 2, "NotFoundError", RuntimeError)
OutOfRangeError = _typed("OutOfRangeError", 3, "OutOfRangeError", IndexError)
AlreadyExistsError = _typed("AlreadyExistsError", 4, "AlreadyExistsError", RuntimeError)
ResourceExhaustedError = _typed("ResourceExhaustedError", 5, "ResourceExhaustedError", MemoryError)
PreconditionNotMetError = _typed("PreconditionNotMetError", 6, "PreconditionNotMetError", RuntimeError)
PermissionDeniedError = _typed("PermissionDeniedError", 7, "PermissionDeniedError", RuntimeError)
ExecutionTimeoutError = _typed("ExecutionTimeoutError", 8, "ExecutionTimeout", RuntimeError)
UnimplementedError = _typed("UnimplementedError", 9, "UnimplementedError", NotImplementedError)
UnavailableError = _typed("UnavailableError", 10, "UnavailableError", RuntimeError)
FatalError = _typed("FatalError", 11, "FatalError", SystemError)
ExternalError = _typed("ExternalError", 12, "ExternalError", OSError)
InvalidTypeError = _typed("InvalidTypeError", 13, "InvalidTypeError", TypeError)

BY_CODE = {c.code: c for c in (InvalidArgumentError, NotFoundError, OutOfRangeError, AlreadyExistsError,
                               ResourceExhaustedError, PreconditionNotMetError, PermissionDeniedError,
                               ExecutionTimeoutError, UnimplementedError, UnavailableError, FatalError, ExternalError,
                               InvalidTypeError)}


def enforce(condition, error_cls=PreconditionNotMetError, message=""):
    """``PADDLE_ENFORCE``: raise ``error_cls(message)`` unless ``condition`` holds."""
    if not condition:
        raise error_cls(message)


def enforce_eq(a, b, error_cls=InvalidArgumentError, message=""):
    if a != b:
        raise error_cls(f"{message} (expected {a!r} == {b!r})".strip())


# launcher return codes of the native kernel entry points (csrc/kernels/host_utils.h) -> typed errors.  The launch
# errors stay ``RuntimeError`` instances as well: callers written against the plain launcher check keep working.
class _LaunchError(RuntimeError):
    pass


LaunchInvalidArgument = type("LaunchInvalidArgument", (InvalidArgumentError, _LaunchError), {})
LaunchOutOfRange = type("LaunchOutOfRange", (OutOfRangeError, _LaunchError), {})
LaunchExternal = type("LaunchExternal", (ExternalError, _LaunchError), {})
LAUNCH_ERROR_CLASSES = {-1: LaunchInvalidArgument, -2: LaunchInvalidArgument, -3: LaunchExternal, -4: LaunchExternal,
                        -5: LaunchOutOfRange}
