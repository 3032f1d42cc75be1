"""``paddle.vision``"""
from . import datasets, models, ops, transforms  # noqa: F401
from .models import *  # noqa: F401,F403

from . import image  # noqa: E402,F401
from .image import get_image_backend, image_load, set_image_backend  # noqa: E402,F401
