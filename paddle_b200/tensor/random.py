"""Random tensor API + global generator control (python/paddle/tensor/random.py,
python/paddle/framework/random.py)."""
from __future__ import annotations

import torch

from .._core import dtype as _dt
from .._core.tensor import as_tensor
from .creation import _shape


def seed(s: int):
    torch.manual_seed(int(s))
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(int(s))
    return torch.default_generator


def get_rng_state(device=None):
    if torch.cuda.is_available() and (device is None or str(device).startswith(("gpu", "cuda"))):
        return [torch.cuda.get_rng_state(i) for i in range(torch.cuda.device_count())]
    return [torch.get_rng_state()]


def set_rng_state(state, device=None):
    if torch.cuda.is_available() and (device is None or str(device).startswith(("gpu", "cuda"))):
        for i, s in enumerate(state):
            torch.cuda.set_rng_state(s, i)
    else:
        torch.set_rng_state(state[0])


def get_cuda_rng_state():
    return [torch.cuda.get_rng_state(i) for i in range(torch.cuda.device_count())] if torch.cuda.is_available() else []


def set_cuda_rng_state(state):
    for i, s in enumerate(state):
        torch.cuda.set_rng_state(s, i)


def _td(dtype):
    return _dt.to_torch(dtype) or _dt.get_default_dtype()


def rand(shape, dtype=None, name=None):
    return as_tensor(torch.rand(_shape(shape), dtype=_td(dtype), device=_dt.default_device()))


def randn(shape, dtype=None, name=None):
    return as_tensor(torch.randn(_shape(shape), dtype=_td(dtype), device=_dt.default_device()))


standard_normal = randn


def normal(mean=0.0, std=1.0, shape=None, name=None):
    if isinstance(mean, torch.Tensor) or isinstance(std, torch.Tensor):
        return as_tensor(torch.normal(mean, std))
    return as_tensor(torch.empty(_shape(shape), dtype=_dt.get_default_dtype(), device=_dt.default_device()).normal_(mean, std))


def uniform(shape, dtype=None, min=-1.0, max=1.0, seed=0, name=None):
    return as_tensor(torch.empty(_shape(shape), dtype=_td(dtype), device=_dt.default_device()).uniform_(min, max))


def randint(low=0, high=None, shape=(1,), dtype=None, name=None):
    if high is None:
        low, high = 0, low
    return as_tensor(torch.randint(int(low), int(high), _shape(shape), dtype=_dt.to_torch(dtype) or torch.int64,
                                   device=_dt.default_device()))


def randint_like(x, low=0, high=None, dtype=None, name=None):
    if high is None:
        low, high = 0, low
    return as_tensor(torch.randint_like(x, int(low), int(high), dtype=_dt.to_torch(dtype)))


def randperm(n, dtype="int64", name=None):
    return as_tensor(torch.randperm(int(n), dtype=_dt.to_torch(dtype), device=_dt.default_device()))


def bernoulli(x, name=None):
    return torch.bernoulli(x)


def multinomial(x, num_samples=1, replacement=False, name=None):
    return torch.multinomial(x, num_samples, replacement)


def poisson(x, name=None):
    return torch.poisson(x)


def exponential_(x, lam=1.0, name=None):
    return x.exponential_(lam)


def uniform_(x, min=-1.0, max=1.0, seed=0, name=None):
    return x.uniform_(min, max)


def normal_(x, mean=0.0, std=1.0, name=None):
    return x.normal_(mean, std)


def standard_gamma(x, name=None):
    return torch._standard_gamma(x)


def binomial(count, prob, name=None):
    return torch.binomial(count.to(prob.dtype), prob).to(torch.int64)
