from ..collective import *  # noqa: F401,F403
from . import stream  # noqa: F401
