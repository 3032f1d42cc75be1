"""``paddle.incubate.multiprocessing``: ``multiprocessing`` with tensors passed between processes through shared
memory (python/paddle/incubate/multiprocessing/reductions.py); the reducers are torch's."""
from multiprocessing import *  # noqa: F401,F403

import torch.multiprocessing as _tmp

__all__ = []


def init_reductions():
    _tmp.reductions.init_reductions()
    from ..._core.tensor import EagerParamBase, Tensor
    from multiprocessing.reduction import ForkingPickler
    import torch
    for cls in (Tensor, EagerParamBase):
        ForkingPickler.register(cls, lambda t: _tmp.reductions.reduce_tensor(t.as_subclass(torch.Tensor)))


init_reductions()
