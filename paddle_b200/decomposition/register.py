"""Rule registry (python/paddle/decomposition/register.py:41-80)."""
from __future__ import annotations

_RULES = {}


def _norm(op_type: str) -> str:
    """``pd_op.softmax`` and ``softmax`` name the same operator."""
    return op_type.split(".", 1)[1] if op_type.startswith("pd_op.") else op_type


def register_decomp(op_type):
    """Decorator: ``fn(*args, **kwargs)`` computes operator ``op_type`` from primitive operators only.  Its signature
    is the signature of the recorded call it replaces."""
    if not isinstance(op_type, str):
        raise TypeError(f"op_type must be a str, got {type(op_type).__name__}")

    def wrap(fn):
        key = _norm(op_type)
        if key in _RULES:
            raise ValueError(f"a decomposition rule for {op_type!r} is already registered")
        _RULES[key] = fn
        return fn
    return wrap


def get_decomp_rule(op_type):
    return _RULES.get(_norm(op_type))


def registered_ops():
    return sorted(_RULES)
