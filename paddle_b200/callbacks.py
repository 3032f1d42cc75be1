"""``paddle.callbacks`` (python/paddle/callbacks.py): the callback classes of ``paddle.Model``."""
from .hapi.callbacks import (Callback, EarlyStopping, LRScheduler, ModelCheckpoint, ProgBarLogger, ReduceLROnPlateau, VisualDL,  # noqa: F401
                             WandbCallback)

__all__ = ["Callback", "ProgBarLogger", "ModelCheckpoint", "VisualDL", "LRScheduler", "EarlyStopping", "ReduceLROnPlateau", "WandbCallback"]
