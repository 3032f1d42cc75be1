"""``paddle.autograd.py_layer`` module path (python/paddle/autograd/py_layer.py)."""
from . import PyLayer, PyLayerContext  # noqa: F401
