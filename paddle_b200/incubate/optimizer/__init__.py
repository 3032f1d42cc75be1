"""``paddle.incubate.optimizer``: LookAhead (lookahead.py:34), ModelAverage (modelaverage.py:38), LBFGS re-export."""
from __future__ import annotations

import torch

from ..._core.tensor import as_tensor


class LookAhead:
    """Every ``k`` fast steps the slow weights move ``alpha`` of the way to the fast weights and the fast weights are
    reset to them."""

    def __init__(self, inner_optimizer, alpha=0.5, k=5, name=None):
        assert inner_optimizer is not None and 0.0 <= alpha <= 1.0 and isinstance(k, int) and k > 0
        self.inner_optimizer, self.alpha, self.k = inner_optimizer, alpha, k
        self._step = 0
        self._slow = {}

    def step(self):
        self.inner_optimizer.step()
        self._step += 1
        with torch.no_grad():
            for p in self.inner_optimizer._parameter_list:
                if p.name not in self._slow:
                    self._slow[p.name] = p.detach().clone()
            if self._step % self.k == 0:
                for p in self.inner_optimizer._parameter_list:
                    slow = self._slow[p.name]
                    slow.add_(p.detach() - slow, alpha=self.alpha)
                    p.copy_(slow)

    def minimize(self, loss, startup_program=None, parameters=None, no_grad_set=None):
        loss.backward()
        self.step()
        return None, None

    def clear_grad(self, set_to_zero=True):
        self.inner_optimizer.clear_grad(set_to_zero)

    def state_dict(self):
        sd = self.inner_optimizer.state_dict()
        sd.update({f"{n}_slow_0": as_tensor(t) for n, t in self._slow.items()})
        return sd

    def __getattr__(self, item):
        return getattr(self.inner_optimizer, item)


class ModelAverage:
    """Running average of parameters over a sliding window; ``apply()`` swaps the averages in (context manager),
    ``restore()`` swaps the trained values back."""

    def __init__(self, average_window_rate, parameters=None, min_average_window=10000, max_average_window=10000, name=None):
        self.rate, self.min_w, self.max_w = average_window_rate, min_average_window, max_average_window
        self._params = list(parameters)
        self._sum = {p.name: torch.zeros_like(p.detach(), dtype=torch.float32) for p in self._params}
        self._n = 0
        self._backup = None

    def step(self):
        with torch.no_grad():
            for p in self._params:
                self._sum[p.name] += p.detach().float()
        self._n += 1
        if self._n > self.max_w:
            for k in self._sum:
                self._sum[k] *= 0.5
            self._n = self._n // 2

    def minimize(self, loss, *a, **k):
        self.step()

    def apply(self, executor=None, need_restore=True):
        ma = self

        class _Ctx:
            def __enter__(self_inner):
                ma._backup = {p.name: p.detach().clone() for p in ma._params}
                with torch.no_grad():
                    for p in ma._params:
                        p.copy_((ma._sum[p.name] / max(ma._n, 1)).to(p.dtype))

            def __exit__(self_inner, *exc):
                if need_restore:
                    ma.restore()
        return _Ctx()

    def restore(self, executor=None):
        if self._backup is not None:
            with torch.no_grad():
                for p in self._params:
                    p.copy_(self._backup[p.name])
            self._backup = None


from ...optimizer.extras import LBFGS  # noqa: E402,F401
from . import functional  # noqa: E402,F401
