"""``paddle.framework``: save/load, RNG seeding, dtype defaults, flags."""
from .._core.dtype import get_default_dtype, set_default_dtype  # noqa: F401
from ..tensor.random import get_cuda_rng_state, get_rng_state, seed, set_cuda_rng_state, set_rng_state  # noqa: F401
from .flags import get_flags, set_flags  # noqa: F401
from .io import async_save, clear_async_save_task_queue, load, save  # noqa: F401
from . import io, random  # noqa: F401


def __getattr__(name):
    # ``paddle.framework.ParamAttr`` and friends live with the layers; resolved lazily to keep imports acyclic
    if name in ("ParamAttr", "WeightNormParamAttr"):
        from ..nn.layer import layers
        return getattr(layers, name, getattr(__import__("paddle_b200").nn, name))
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
