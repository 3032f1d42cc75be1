"""``paddle.utils.unique_name`` (python/paddle/utils/unique_name.py)."""
from .._core.unique_name import generate, guard, switch  # noqa: F401

__all__ = ["generate", "switch", "guard"]
