"""``paddle.hapi``: the high-level ``paddle.Model`` API (python/paddle/hapi/: model.py, callbacks.py, model_summary.py,
dynamic_flops.py, progressbar.py, logger.py)."""
from . import callbacks, dynamic_flops, logger, model, model_summary, progressbar  # noqa: F401
from .callbacks import (Callback, CallbackList, EarlyStopping, LRScheduler, ModelCheckpoint, ProgBarLogger, ReduceLROnPlateau, VisualDL,
                        WandbCallback, config_callbacks)
from .dynamic_flops import flops
from .model import Model
from .model_summary import summary

__all__ = ["Model", "summary", "flops", "callbacks"]
