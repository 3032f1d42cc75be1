"""``paddle.hapi.callbacks`` (python/paddle/hapi/callbacks.py): the callback classes live in ``paddle.callbacks``."""
from .. import callbacks as _cb

__all__ = [n for n in dir(_cb) if not n.startswith("_") and isinstance(getattr(_cb, n), type)]
globals().update({n: getattr(_cb, n) for n in __all__})
