"""RNG state tracker for tensor parallelism (python/paddle/distributed/fleet/layers/mpu/random.py):
named generator states so that dropout inside a tensor-parallel region draws different numbers on each
mp rank while dropout outside draws the same."""
from __future__ import annotations

import contextlib

import torch

MODEL_PARALLEL_RNG = "model_parallel_rng"


class RNGStatesTracker:
    def __init__(self):
        self.states_ = {}
        self.seeds_ = set()

    def reset(self):
        self.states_.clear()
        self.seeds_.clear()

    def _get(self):
        return torch.cuda.get_rng_state() if torch.cuda.is_available() else torch.get_rng_state()

    def _set(self, s):
        (torch.cuda.set_rng_state if torch.cuda.is_available() else torch.set_rng_state)(s)

    def add(self, name, seed):
        if seed in self.seeds_:
            raise ValueError(f"seed {seed} already exists")
        if name in self.states_:
            raise ValueError(f"state {name} already exists")
        self.seeds_.add(seed)
        orig = self._get()
        (torch.cuda.manual_seed if torch.cuda.is_available() else torch.manual_seed)(seed)
        self.states_[name] = self._get()
        self._set(orig)

    def get_states_tracker(self):
        return dict(self.states_)

    def set_states_tracker(self, states):
        self.states_ = dict(states)

    @contextlib.contextmanager
    def rng_state(self, name=MODEL_PARALLEL_RNG):
        if name not in self.states_:
            raise ValueError(f"state {name} does not exist")
        orig = self._get()
        self._set(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = self._get()
            self._set(orig)


RNG_STATE_TRACKER = RNGStatesTracker()


def get_rng_state_tracker():
    return RNG_STATE_TRACKER


def model_parallel_random_seed(seed=None):
    from ... import fleet
    import random as _r
    hcg = fleet.get_hybrid_communicate_group()
    rank = hcg.get_model_parallel_rank()
    if seed:
        global_seed, local_seed = seed, seed * 1024 + rank * 100
    else:
        global_seed = 100 + hcg.get_data_parallel_rank() * 0 + 7
        local_seed = 1024 + global_seed + rank * 100
    RNG_STATE_TRACKER.reset()
    RNG_STATE_TRACKER.add(MODEL_PARALLEL_RNG, local_seed)
    import paddle_b200
    paddle_b200.seed(global_seed)


def determinate_seed(rng_name):
    return 0


def dropout(x, p=0.5, axis=None, rng_name=None, training=True, mode="upscale_in_train", name=None):
    from .....nn import functional as F
    if rng_name is None:
        return F.dropout(x, p, axis, training, mode)
    with RNG_STATE_TRACKER.rng_state(rng_name):
        return F.dropout(x, p, axis, training, mode)
