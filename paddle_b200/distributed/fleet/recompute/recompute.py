"""``paddle.distributed.fleet.recompute.recompute`` module path (python/paddle/distributed/fleet/recompute/recompute.py)."""
from . import RecomputeFunction, recompute, recompute_sequential  # noqa: F401

import contextlib
import logging

import torch

logger = logging.getLogger(__name__)


def detach_variable(inputs):
    """Detached copies of the tensors among ``inputs`` (tuples of tensors element-wise) that keep their
    ``stop_gradient`` flag; everything else passes through (recompute.py:62)."""
    def one(t):
        d = t.detach()
        d.requires_grad_(t.requires_grad)
        return d
    out = []
    for inp in inputs:
        if isinstance(inp, torch.Tensor):
            out.append(one(inp))
        elif type(inp) is tuple and inp and isinstance(inp[0], torch.Tensor):
            out.append(tuple(one(i) for i in inp))
        else:
            out.append(inp)
    return tuple(out)


def check_recompute_necessary(inputs):
    """Warns when no input of a recompute block needs a gradient: then nothing is re-run in backward and the block
    only costs memory bookkeeping (recompute.py:98)."""
    flags = []
    for inp in inputs:
        for t in (inp if type(inp) is tuple else (inp,)):
            if isinstance(t, torch.Tensor):
                flags.append(not t.requires_grad)
    if flags and all(flags):
        logger.warning("[Recompute]: None of the inputs to current recompute block need grad, "
                       "therefore there is NO need to recompute this block in backward !")
    return not (flags and all(flags))


@contextlib.contextmanager
def switch_rng_state_tracker(rng_state, tracker):
    """Runs the block under the saved global RNG state and the saved named states of the model-parallel RNG tracker,
    then restores both (recompute.py:116)."""
    from ..layers.mpu.random import get_rng_state_tracker
    import paddle_b200 as paddle
    orig_state = paddle.get_rng_state()
    orig_tracker = get_rng_state_tracker().get_states_tracker()
    paddle.set_rng_state(rng_state)
    get_rng_state_tracker().set_states_tracker(tracker)
    try:
        yield
    finally:
        paddle.set_rng_state(orig_state)
        get_rng_state_tracker().set_states_tracker(orig_tracker)
