"""Parameter initializers (python/paddle/nn/initializer/).  Each is a callable applied in place."""
from __future__ import annotations

import math

import numpy as np
import torch

_GLOBAL = {"weight": None, "bias": None}


def set_global_initializer(weight_init, bias_init=None):
    _GLOBAL["weight"], _GLOBAL["bias"] = weight_init, bias_init


def _global_initializer(is_bias):
    return _GLOBAL["bias" if is_bias else "weight"]


def _fans(t):
    shape = t.shape
    if len(shape) == 0:
        return 1, 1
    if len(shape) == 1:
        return shape[0], shape[0]
    if len(shape) == 2:  # Paddle Linear weight is [in, out]
        return shape[0], shape[1]
    rf = int(np.prod(shape[2:]))
    return shape[1] * rf, shape[0] * rf


class Initializer:
    def __call__(self, param, block=None):
        raise NotImplementedError


class Constant(Initializer):
    def __init__(self, value=0.0):
        self.value = value

    def __call__(self, param, block=None):
        with torch.no_grad():
            param.fill_(self.value)
        return param


class Normal(Initializer):
    def __init__(self, mean=0.0, std=1.0, name=None):
        self.mean, self.std = mean, std

    def __call__(self, param, block=None):
        with torch.no_grad():
            if param.dtype in (torch.bfloat16, torch.float16):
                param.copy_(torch.empty(param.shape, dtype=torch.float32, device=param.device).normal_(self.mean, self.std))
            else:
                param.normal_(self.mean, self.std)
        return param


class TruncatedNormal(Initializer):
    def __init__(self, mean=0.0, std=1.0, a=-2.0, b=2.0, name=None):
        self.mean, self.std, self.a, self.b = mean, std, a, b

    def __call__(self, param, block=None):
        with torch.no_grad():
            t = torch.empty(param.shape, dtype=torch.float32, device=param.device)
            torch.nn.init.trunc_normal_(t, self.mean, self.std, self.mean + self.a * self.std, self.mean + self.b * self.std)
            param.copy_(t)
        return param


class Uniform(Initializer):
    def __init__(self, low=-1.0, high=1.0, name=None):
        self.low, self.high = low, high

    def __call__(self, param, block=None):
        with torch.no_grad():
            t = torch.empty(param.shape, dtype=torch.float32, device=param.device).uniform_(self.low, self.high)
            param.copy_(t)
        return param


class XavierUniform(Initializer):
    def __init__(self, fan_in=None, fan_out=None, gain=1.0, name=None):
        self.fan_in, self.fan_out, self.gain = fan_in, fan_out, gain

    def __call__(self, param, block=None):
        fi, fo = _fans(param)
        fi, fo = self.fan_in or fi, self.fan_out or fo
        limit = self.gain * math.sqrt(6.0 / (fi + fo))
        return Uniform(-limit, limit)(param)


class XavierNormal(Initializer):
    def __init__(self, fan_in=None, fan_out=None, gain=1.0, name=None):
        self.fan_in, self.fan_out, self.gain = fan_in, fan_out, gain

    def __call__(self, param, block=None):
        fi, fo = _fans(param)
        fi, fo = self.fan_in or fi, self.fan_out or fo
        return Normal(0.0, self.gain * math.sqrt(2.0 / (fi + fo)))(param)


class KaimingUniform(Initializer):
    def __init__(self, fan_in=None, negative_slope=0.0, nonlinearity="relu", mode="fan_in"):
        self.fan_in, self.negative_slope, self.nonlinearity, self.mode = fan_in, negative_slope, nonlinearity, mode

    def __call__(self, param, block=None):
        fi, fo = _fans(param)
        fan = self.fan_in or (fi if self.mode == "fan_in" else fo)
        gain = torch.nn.init.calculate_gain(self.nonlinearity, self.negative_slope) if self.nonlinearity in (
            "relu", "leaky_relu", "tanh", "sigmoid", "linear", "selu") else math.sqrt(2.0)
        limit = gain * math.sqrt(3.0 / fan)
        return Uniform(-limit, limit)(param)


class KaimingNormal(KaimingUniform):
    def __call__(self, param, block=None):
        fi, fo = _fans(param)
        fan = self.fan_in or (fi if self.mode == "fan_in" else fo)
        gain = torch.nn.init.calculate_gain(self.nonlinearity, self.negative_slope) if self.nonlinearity in (
            "relu", "leaky_relu", "tanh", "sigmoid", "linear", "selu") else math.sqrt(2.0)
        return Normal(0.0, gain / math.sqrt(fan))(param)


MSRAInitializer = KaimingNormal


class Assign(Initializer):
    def __init__(self, value, name=None):
        self.value = value

    def __call__(self, param, block=None):
        v = self.value if isinstance(self.value, torch.Tensor) else torch.as_tensor(np.asarray(self.value))
        with torch.no_grad():
            v = v.to(param.dtype)
            # a value with fewer elements than the parameter is broadcast (Assign(np.array([2, 2])) fills a 2 x 2 weight)
            param.copy_(v.reshape(param.shape) if v.numel() == param.numel() else torch.broadcast_to(v, param.shape))
        return param


NumpyArrayInitializer = Assign


class Orthogonal(Initializer):
    def __init__(self, gain=1.0, name=None):
        self.gain = gain

    def __call__(self, param, block=None):
        with torch.no_grad():
            t = torch.empty(param.shape, dtype=torch.float32, device=param.device)
            torch.nn.init.orthogonal_(t, self.gain)
            param.copy_(t)
        return param


class Dirac(Initializer):
    def __init__(self, groups=1, name=None):
        self.groups = groups

    def __call__(self, param, block=None):
        with torch.no_grad():
            t = torch.empty(param.shape, dtype=torch.float32, device=param.device)
            torch.nn.init.dirac_(t, self.groups)
            param.copy_(t)
        return param


class Bilinear(Initializer):
    def __call__(self, param, block=None):
        shape = param.shape
        f = math.ceil(shape[3] / 2.0)
        c = (2 * f - 1 - f % 2) / (2.0 * f)
        w = np.zeros(int(np.prod(shape)), dtype=np.float32)
        for i in range(w.size):
            x, y = i % shape[3], (i // shape[3]) % shape[2]
            w[i] = (1 - abs(x / f - c)) * (1 - abs(y / f - c))
        return Assign(w.reshape(shape))(param)


def calculate_gain(nonlinearity, param=None):
    return torch.nn.init.calculate_gain(nonlinearity, param)
