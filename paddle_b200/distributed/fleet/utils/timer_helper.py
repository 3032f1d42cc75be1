"""Named timers for training loops (python/paddle/distributed/fleet/utils/timer_helper.py): ``get_timers()``,
``set_timers()``, ``timers("name").start()/stop()``, ``timers.log(names)``.  GPU work is timed with CUDA events, so
``elapsed`` reports device time without forcing a synchronisation at every ``stop``."""
from __future__ import annotations

import time

import torch

_GLOBAL_TIMERS = None


class _Timer:
    def __init__(self, name):
        self.name, self.elapsed_, self.started_ = name, 0.0, False
        self._pairs = []
        self._t0 = None

    def start(self):
        assert not self.started_, "timer has already started"
        if torch.cuda.is_available():
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._t0 = e
        else:
            self._t0 = time.time()
        self.started_ = True

    def stop(self):
        assert self.started_, "timer is not started."
        if torch.cuda.is_available():
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pairs.append((self._t0, e))
        else:
            self.elapsed_ += time.time() - self._t0
        self.started_ = False

    def reset(self):
        self.elapsed_, self.started_, self._pairs = 0.0, False, []

    def elapsed(self, reset=True):
        started = self.started_
        if started:
            self.stop()
        if self._pairs:
            torch.cuda.synchronize()
            self.elapsed_ += sum(a.elapsed_time(b) for a, b in self._pairs) / 1e3
            self._pairs = []
        out = self.elapsed_
        if reset:
            self.reset()
        if started:
            self.start()
        return out


class Timers:
    def __init__(self):
        self.timers = {}

    def __call__(self, name):
        if name not in self.timers:
            self.timers[name] = _Timer(name)
        return self.timers[name]

    def log(self, names, normalizer=1.0, reset=True):
        assert normalizer > 0.0
        s = "time (ms)"
        for n in names:
            s += f" | {n}: {self.timers[n].elapsed(reset=reset) * 1000.0 / normalizer:.2f}"
        print(s, flush=True)
        return s


def is_timer_initialized():
    return _GLOBAL_TIMERS is not None


def get_timers():
    return _GLOBAL_TIMERS


def set_timers():
    global _GLOBAL_TIMERS
    _GLOBAL_TIMERS = Timers()
