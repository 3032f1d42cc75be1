"""``paddle.tensor``: functional tensor API.  Everything here is also re-exported from the package
root and bound as methods of :class:`paddle_b200.Tensor`."""
from . import creation, linalg, manipulation, math, random  # noqa: F401
from .creation import *  # noqa: F401,F403
from .linalg import *  # noqa: F401,F403
from .manipulation import *  # noqa: F401,F403
from .math import *  # noqa: F401,F403
from .random import *  # noqa: F401,F403
