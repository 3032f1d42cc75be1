"""``paddle.nn``"""
from . import functional, initializer  # noqa: F401
from .clip import ClipGradByGlobalNorm, ClipGradByNorm, ClipGradByValue  # noqa: F401
from .layer.common import *  # noqa: F401,F403
from .layer.layers import Layer, ParamAttr  # noqa: F401
from . import utils  # noqa: F401
