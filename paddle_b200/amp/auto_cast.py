"""``paddle.amp.auto_cast`` module path (python/paddle/amp/auto_cast.py)."""
from . import amp_state, auto_cast, decorate, is_bfloat16_supported, is_float16_supported  # noqa: F401

amp_guard = auto_cast
amp_decorate = decorate
