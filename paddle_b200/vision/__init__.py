"""``paddle.vision``"""
from . import datasets, models, ops, transforms  # noqa: F401
from .models import *  # noqa: F401,F403

_backend = "pil"


def set_image_backend(backend):
    global _backend
    if backend not in ("pil", "cv2", "tensor"):
        raise ValueError(f"Expected backend are one of ['pil', 'cv2', 'tensor'], but got {backend}")
    _backend = backend


def get_image_backend():
    return _backend


def image_load(path, backend=None):
    from PIL import Image
    return Image.open(path)
