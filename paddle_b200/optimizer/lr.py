"""Learning-rate schedulers (python/paddle/optimizer/lr.py).  ``scheduler()`` returns the current
value, ``step()`` advances ``last_epoch``; ``state_dict`` keeps ``last_epoch`` and ``last_lr``."""
from __future__ import annotations

import math


class LRScheduler:
    def __init__(self, learning_rate=0.1, last_epoch=-1, verbose=False):
        self.base_lr = float(learning_rate)
        self.last_lr = float(learning_rate)
        self.last_epoch = last_epoch
        self.verbose = verbose
        self.step()

    def __call__(self):
        return self.last_lr

    def step(self, epoch=None):
        self.last_epoch = self.last_epoch + 1 if epoch is None else epoch
        self.last_lr = float(self.get_lr())

    def get_lr(self):
        raise NotImplementedError

    def state_dict(self):
        return {k: v for k, v in self.__dict__.items()
                if isinstance(v, (int, float, bool, str, list, tuple)) and k not in ("verbose",)}

    def set_state_dict(self, sd):
        for k, v in sd.items():
            if k in self.__dict__:
                self.__dict__[k] = v

    set_dict = set_state_dict
    state_keys = lambda self: None  # noqa: E731


class NoamDecay(LRScheduler):
    def __init__(self, d_model, warmup_steps, learning_rate=1.0, last_epoch=-1, verbose=False):
        self.d_model, self.warmup_steps = d_model, warmup_steps
        super().__init__(learning_rate, last_epoch, verbose)

    def get_lr(self):
        e = max(self.last_epoch, 1)
        return self.base_lr * self.d_model ** -0.5 * min(e ** -0.5, e * self.warmup_steps ** -1.5)


class PiecewiseDecay(LRScheduler):
    def __init__(self, boundaries, values, last_epoch=-1, verbose=False):
        self.boundaries, self.values = list(boundaries), list(values)
        super().__init__(values[0], last_epoch, verbose)

    def get_lr(self):
        for b, v in zip(self.boundaries, self.values):
            if self.last_epoch < b:
                return v
        return self.values[len(self.boundaries)]


class NaturalExpDecay(LRScheduler):
    def __init__(self, learning_rate, gamma, last_epoch=-1, verbose=False):
        self.gamma = gamma
        super().__init__(learning_rate, last_epoch, verbose)

    def get_lr(self):
        return self.base_lr * math.exp(-self.gamma * self.last_epoch)


class InverseTimeDecay(NaturalExpDecay):
    def get_lr(self):
        return self.base_lr / (1 + self.gamma * self.last_epoch)


class ExponentialDecay(NaturalExpDecay):
    def get_lr(self):
        return self.base_lr * self.gamma ** self.last_epoch


class PolynomialDecay(LRScheduler):
    def __init__(self, learning_rate, decay_steps, end_lr=0.0001, power=1.0, cycle=False, last_epoch=-1, verbose=False):
        self.decay_steps, self.end_lr, self.power, self.cycle = decay_steps, end_lr, power, cycle
        super().__init__(learning_rate, last_epoch, verbose)

    def get_lr(self):
        t, n = self.last_epoch, self.decay_steps
        if self.cycle:
            n = n * max(1.0, math.ceil(t / n))
        else:
            t = min(t, n)
        return (self.base_lr - self.end_lr) * (1 - t / n) ** self.power + self.end_lr


class LinearWarmup(LRScheduler):
    def __init__(self, learning_rate, warmup_steps, start_lr, end_lr, last_epoch=-1, verbose=False):
        self.inner = learning_rate
        self.warmup_steps, self.start_lr, self.end_lr = warmup_steps, start_lr, end_lr
        super().__init__(end_lr if isinstance(learning_rate, LRScheduler) else learning_rate, last_epoch, verbose)

    def get_lr(self):
        if self.last_epoch < self.warmup_steps:
            return (self.end_lr - self.start_lr) * self.last_epoch / self.warmup_steps + self.start_lr
        if isinstance(self.inner, LRScheduler):
            self.inner.step(self.last_epoch - self.warmup_steps)
            return self.inner()
        return float(self.inner)

    def state_dict(self):
        sd = super().state_dict()
        if isinstance(self.inner, LRScheduler):
            sd["LinearWarmup_LR"] = self.inner.state_dict()
        return sd

    def set_state_dict(self, sd):
        sd = dict(sd)
        inner = sd.pop("LinearWarmup_LR", None)
        super().set_state_dict(sd)
        if inner is not None and isinstance(self.inner, LRScheduler):
            self.inner.set_state_dict(inner)


class LinearLR(LRScheduler):
    """Multiplies the rate by a factor that moves linearly from ``start_factor`` to ``end_factor`` over ``total_steps``."""

    def __init__(self, learning_rate, total_steps, start_factor=1.0 / 3, end_factor=1.0, last_epoch=-1, verbose=False):
        if start_factor > 1.0 or start_factor <= 0:
            raise ValueError(f"`start_factor` must be greater than 0 and less or equal to 1, but got {start_factor}")
        if end_factor > 1.0 or end_factor < 0:
            raise ValueError(f"`end_factor` must be greater than 0 and less than 1, but got {end_factor}")
        if total_steps <= 0:
            raise ValueError(f"`total_steps` must be greater than 0, but got {total_steps}")
        self.start_factor, self.end_factor, self.total_steps = start_factor, end_factor, total_steps
        super().__init__(learning_rate, last_epoch, verbose)

    def get_lr(self):
        t = min(max(self.last_epoch, 0), self.total_steps)
        return self.base_lr * (self.start_factor + (self.end_factor - self.start_factor) * t / self.total_steps)


class StepDecay(LRScheduler):
    def __init__(self, learning_rate, step_size, gamma=0.1, last_epoch=-1, verbose=False):
        self.step_size, self.gamma = step_size, gamma
        super().__init__(learning_rate, last_epoch, verbose)

    def get_lr(self):
        return self.base_lr * self.gamma ** (self.last_epoch // self.step_size)


class MultiStepDecay(LRScheduler):
    def __init__(self, learning_rate, milestones, gamma=0.1, last_epoch=-1, verbose=False):
        self.milestones, self.gamma = list(milestones), gamma
        super().__init__(learning_rate, last_epoch, verbose)

    def get_lr(self):
        return self.base_lr * self.gamma ** sum(1 for m in self.milestones if self.last_epoch >= m)


class LambdaDecay(LRScheduler):
    def __init__(self, learning_rate, lr_lambda, last_epoch=-1, verbose=False):
        self.lr_lambda = lr_lambda
        super().__init__(learning_rate, last_epoch, verbose)

    def get_lr(self):
        return self.base_lr * self.lr_lambda(self.last_epoch)


class MultiplicativeDecay(LambdaDecay):
    def get_lr(self):
        lr = self.base_lr
        for e in range(1, self.last_epoch + 1):
            lr *= self.lr_lambda(e)
        return lr


class CosineAnnealingDecay(LRScheduler):
    def __init__(self, learning_rate, T_max, eta_min=0, last_epoch=-1, verbose=False):
        self.T_max, self.eta_min = T_max, eta_min
        super().__init__(learning_rate, last_epoch, verbose)

    def get_lr(self):
        return self.eta_min + (self.base_lr - self.eta_min) * (1 + math.cos(math.pi * self.last_epoch / self.T_max)) / 2


class CosineAnnealingWarmRestarts(LRScheduler):
    def __init__(self, learning_rate, T_0, T_mult=1, eta_min=0, last_epoch=-1, verbose=False):
        self.T_0, self.T_mult, self.eta_min = T_0, T_mult, eta_min
        super().__init__(learning_rate, last_epoch, verbose)

    def get_lr(self):
        t, ti = self.last_epoch, self.T_0
        while t >= ti:
            t -= ti
            ti *= self.T_mult
        return self.eta_min + (self.base_lr - self.eta_min) * (1 + math.cos(math.pi * t / ti)) / 2


class OneCycleLR(LRScheduler):
    def __init__(self, max_learning_rate, total_steps, divide_factor=25.0, end_learning_rate=0.0001, phase_pct=0.3,
                 anneal_strategy="cos", three_phase=False, last_epoch=-1, verbose=False):
        self.max_lr, self.total_steps, self.end_lr, self.phase_pct = max_learning_rate, total_steps, end_learning_rate, phase_pct
        self.init_lr = max_learning_rate / divide_factor
        self.anneal = anneal_strategy
        super().__init__(self.init_lr, last_epoch, verbose)

    def _interp(self, a, b, pct):
        return b + (a - b) / 2 * (math.cos(math.pi * pct) + 1) if self.anneal == "cos" else (b - a) * pct + a

    def get_lr(self):
        up = self.phase_pct * self.total_steps - 1
        t = min(self.last_epoch, self.total_steps - 1)
        if t <= up:
            return self._interp(self.init_lr, self.max_lr, t / max(up, 1))
        return self._interp(self.max_lr, self.end_lr, (t - up) / max(self.total_steps - 1 - up, 1))


class CyclicLR(LRScheduler):
    def __init__(self, base_learning_rate, max_learning_rate, step_size_up, step_size_down=None, mode="triangular",
                 exp_gamma=1.0, scale_fn=None, scale_mode="cycle", last_epoch=-1, verbose=False):
        self.max_lr, self.up = max_learning_rate, step_size_up
        self.down = step_size_down or step_size_up
        self.mode, self.exp_gamma = mode, exp_gamma
        super().__init__(base_learning_rate, last_epoch, verbose)

    def get_lr(self):
        total = self.up + self.down
        cycle = 1 + self.last_epoch // total
        pos = self.last_epoch % total
        pct = pos / self.up if pos <= self.up else 1 - (pos - self.up) / self.down
        scale = {"triangular": 1.0, "triangular2": 1 / 2 ** (cycle - 1), "exp_range": self.exp_gamma ** self.last_epoch}[self.mode]
        return self.base_lr + (self.max_lr - self.base_lr) * pct * scale


class ReduceOnPlateau(LRScheduler):
    def __init__(self, learning_rate, mode="min", factor=0.1, patience=10, threshold=1e-4, threshold_mode="rel",
                 cooldown=0, min_lr=0, epsilon=1e-8, verbose=False):
        self.mode, self.factor, self.patience, self.threshold = mode, factor, patience, threshold
        self.threshold_mode, self.cooldown, self.min_lr, self.epsilon = threshold_mode, cooldown, min_lr, epsilon
        self.best, self.num_bad, self.cooldown_counter = None, 0, 0
        self.base_lr = self.last_lr = float(learning_rate)
        self.last_epoch = 0
        self.verbose = verbose

    def step(self, metrics=None, epoch=None):
        self.last_epoch += 1
        if metrics is None:
            return
        m = float(metrics)
        if self.best is None:
            better = True
        elif self.mode == "min":
            better = m < (self.best * (1 - self.threshold) if self.threshold_mode == "rel" else self.best - self.threshold)
        else:
            better = m > (self.best * (1 + self.threshold) if self.threshold_mode == "rel" else self.best + self.threshold)
        if better:
            self.best, self.num_bad = m, 0
        else:
            self.num_bad += 1
        if self.cooldown_counter > 0:
            self.cooldown_counter -= 1
            self.num_bad = 0
        if self.num_bad > self.patience:
            new = max(self.last_lr * self.factor, self.min_lr)
            if self.last_lr - new > self.epsilon:
                self.last_lr = new
            self.cooldown_counter, self.num_bad = self.cooldown, 0

    def get_lr(self):
        return self.last_lr


# ------------------------------------------------------------------------------------------- functional (legacy) forms
# python/paddle/optimizer/lr.py:2697-3190: the functions of the older API return scheduler objects in dynamic mode;
# ``step()`` advances them once per optimizer update.
def noam_decay(d_model, warmup_steps, learning_rate=1.0):
    return NoamDecay(d_model, warmup_steps, learning_rate)


def exponential_decay(learning_rate, decay_steps, decay_rate, staircase=False):
    """learning_rate * decay_rate ^ (step / decay_steps); ``staircase`` floors the exponent."""
    def f(step):
        e = step / decay_steps
        return decay_rate ** (math.floor(e) if staircase else e)
    return LambdaDecay(learning_rate, f)


def natural_exp_decay(learning_rate, decay_steps, decay_rate, staircase=False):
    """learning_rate * exp(-decay_rate * step / decay_steps)."""
    def f(step):
        e = step / decay_steps
        return math.exp(-decay_rate * (math.floor(e) if staircase else e))
    return LambdaDecay(learning_rate, f)


def inverse_time_decay(learning_rate, decay_steps, decay_rate, staircase=False):
    """learning_rate / (1 + decay_rate * step / decay_steps)."""
    def f(step):
        e = step / decay_steps
        return 1.0 / (1.0 + decay_rate * (math.floor(e) if staircase else e))
    return LambdaDecay(learning_rate, f)


def polynomial_decay(learning_rate, decay_steps, end_learning_rate=0.0001, power=1.0, cycle=False):
    return PolynomialDecay(learning_rate, decay_steps, end_learning_rate, power, cycle)


def piecewise_decay(boundaries, values):
    return PiecewiseDecay(boundaries, values)


def cosine_decay(learning_rate, step_each_epoch, epochs):
    """learning_rate * 0.5 * (cos(epoch * pi / epochs) + 1) with epoch = floor(step / step_each_epoch)."""
    return LambdaDecay(learning_rate, lambda step: 0.5 * (math.cos(math.floor(step / step_each_epoch) * math.pi / epochs) + 1))


def linear_lr_warmup(learning_rate, warmup_steps, start_lr, end_lr):
    return LinearWarmup(learning_rate, warmup_steps, start_lr, end_lr)
