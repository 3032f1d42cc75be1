"""``paddle.utils.install_check.run_check`` (python/paddle/utils/install_check.py:251)."""
from . import run_check  # noqa: F401

__all__ = ["run_check"]
