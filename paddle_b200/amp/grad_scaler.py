"""``paddle.amp.grad_scaler`` module path (python/paddle/amp/grad_scaler.py)."""
from . import GradScaler  # noqa: F401

AmpScaler = GradScaler
