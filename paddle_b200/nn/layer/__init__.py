from .common import *  # noqa: F401,F403
from .layers import HookRemoveHelper, Layer, ParamAttr  # noqa: F401
