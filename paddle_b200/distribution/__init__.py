"""``paddle.distribution`` (python/paddle/distribution/): probability distributions, transforms, KL registry.
Every class wraps the ``torch.distributions`` object of the same law and exposes Paddle's method names
(``sample(shape)``, ``rsample``, ``log_prob``, ``prob``, ``entropy``, ``kl_divergence``, ``mean``/``variance``)."""
from __future__ import annotations

import torch
import torch.distributions as D

from .._core.tensor import as_tensor

__all__ = ["Distribution", "Normal", "Uniform", "Bernoulli", "Beta", "Binomial", "Categorical", "Cauchy", "Chi2",
           "ContinuousBernoulli", "Dirichlet", "Exponential", "ExponentialFamily", "Gamma", "Geometric", "Gumbel",
           "Independent", "Laplace", "LKJCholesky", "LogNormal", "Multinomial", "MultivariateNormal", "Poisson",
           "StudentT", "TransformedDistribution", "kl_divergence", "register_kl", "Transform", "AbsTransform",
           "AffineTransform", "ChainTransform", "ExpTransform", "IndependentTransform", "PowerTransform",
           "ReshapeTransform", "SigmoidTransform", "SoftmaxTransform", "StackTransform", "StickBreakingTransform",
           "TanhTransform"]


def _t(x):
    if isinstance(x, torch.Tensor):
        return x.as_subclass(torch.Tensor)
    return torch.as_tensor(x, dtype=torch.get_default_dtype()) if isinstance(x, (int, float, list, tuple)) else x


class Distribution:
    _cls = None

    def __init__(self, batch_shape=(), event_shape=()):
        self._batch_shape, self._event_shape = tuple(batch_shape), tuple(event_shape)
        self._d = None

    @classmethod
    def _from(cls, d):
        o = cls.__new__(cls)
        o._d = d
        return o

    batch_shape = property(lambda self: tuple(self._d.batch_shape) if self._d is not None else self._batch_shape)
    event_shape = property(lambda self: tuple(self._d.event_shape) if self._d is not None else self._event_shape)
    mean = property(lambda self: as_tensor(self._d.mean))
    variance = property(lambda self: as_tensor(self._d.variance))
    stddev = property(lambda self: as_tensor(self._d.stddev))

    def sample(self, shape=()):
        with torch.no_grad():
            return as_tensor(self._d.sample(tuple(shape)))

    def rsample(self, shape=()):
        return as_tensor(self._d.rsample(tuple(shape)))

    def log_prob(self, value):
        return as_tensor(self._d.log_prob(_t(value)))

    def prob(self, value):
        return as_tensor(self._d.log_prob(_t(value)).exp())

    probs = prob

    def entropy(self):
        return as_tensor(self._d.entropy())

    def cdf(self, value):
        return as_tensor(self._d.cdf(_t(value)))

    def icdf(self, value):
        return as_tensor(self._d.icdf(_t(value)))

    def kl_divergence(self, other):
        return kl_divergence(self, other)


class ExponentialFamily(Distribution):
    pass


def _make(name, torch_cls, argmap, base=Distribution):
    def __init__(self, *args, **kwargs):
        kwargs.pop("name", None)
        names = list(argmap)
        vals = dict(zip(names, args))
        vals.update(kwargs)
        self._params = vals
        int_args = {"dim", "total_count"} if torch_cls in (D.LKJCholesky, D.Multinomial) else set()
        conv = {argmap[k]: (int(v) if k in int_args and not isinstance(v, torch.Tensor) else
                            (int(v.item()) if k in int_args and v.numel() == 1 else _t(v)))
                for k, v in vals.items() if v is not None}
        self._d = torch_cls(**conv, validate_args=False)
        for k, v in vals.items():
            if not hasattr(type(self), k) or k == "probs":       # the parameter shadows the ``probs(value)`` method alias
                setattr(self, k, as_tensor(_t(v)) if isinstance(_t(v), torch.Tensor) else v)
    return type(name, (base,), {"__init__": __init__})


Normal = _make("Normal", D.Normal, {"loc": "loc", "scale": "scale"}, ExponentialFamily)
Uniform = _make("Uniform", D.Uniform, {"low": "low", "high": "high"})
Bernoulli = _make("Bernoulli", D.Bernoulli, {"probs": "probs"}, ExponentialFamily)
Beta = _make("Beta", D.Beta, {"alpha": "concentration1", "beta": "concentration0"}, ExponentialFamily)
Binomial = _make("Binomial", D.Binomial, {"total_count": "total_count", "probs": "probs"})
Cauchy = _make("Cauchy", D.Cauchy, {"loc": "loc", "scale": "scale"})
Chi2 = _make("Chi2", D.Chi2, {"df": "df"})
ContinuousBernoulli = _make("ContinuousBernoulli", D.ContinuousBernoulli, {"probs": "probs", "lims": "lims"})
Dirichlet = _make("Dirichlet", D.Dirichlet, {"concentration": "concentration"}, ExponentialFamily)
Exponential = _make("Exponential", D.Exponential, {"rate": "rate"}, ExponentialFamily)
Gamma = _make("Gamma", D.Gamma, {"concentration": "concentration", "rate": "rate"}, ExponentialFamily)
Geometric = _make("Geometric", D.Geometric, {"probs": "probs"})
Gumbel = _make("Gumbel", D.Gumbel, {"loc": "loc", "scale": "scale"})
Laplace = _make("Laplace", D.Laplace, {"loc": "loc", "scale": "scale"})
LogNormal = _make("LogNormal", D.LogNormal, {"loc": "loc", "scale": "scale"})
Multinomial = _make("Multinomial", D.Multinomial, {"total_count": "total_count", "probs": "probs"})
MultivariateNormal = _make("MultivariateNormal", D.MultivariateNormal,
                           {"loc": "loc", "covariance_matrix": "covariance_matrix", "precision_matrix": "precision_matrix",
                            "scale_tril": "scale_tril"})
Poisson = _make("Poisson", D.Poisson, {"rate": "rate"})
StudentT = _make("StudentT", D.StudentT, {"df": "df", "loc": "loc", "scale": "scale"})
LKJCholesky = _make("LKJCholesky", D.LKJCholesky, {"dim": "dim", "concentration": "concentration"})


class _GeometricMixin:
    """Number of failures before the first success, k = 0, 1, 2, ... (python/paddle/distribution/geometric.py)."""

    def pmf(self, k):
        p = _t(self.probs)
        return as_tensor(torch.pow(1.0 - p, _t(k)) * p)

    def log_pmf(self, k):
        return as_tensor(torch.log(_t(self.pmf(k))))

    def cdf(self, k):
        p = _t(self.probs)
        return as_tensor(1.0 - torch.pow(1.0 - p, _t(k) + 1))

    def rsample(self, shape=()):
        p = _t(self.probs)
        u = torch.rand(tuple(shape) + tuple(p.shape), dtype=p.dtype).clamp_min(torch.finfo(p.dtype).tiny)
        return as_tensor(torch.floor(torch.log(u) / torch.log1p(-p)))

    def sample(self, shape=()):
        with torch.no_grad():
            return self.rsample(shape)

    def entropy(self):
        p = _t(self.probs)
        return as_tensor(-((1.0 - p) * torch.log(1.0 - p) + p * torch.log(p)) / p)

    def kl_divergence(self, other):
        p, q = _t(self.probs), _t(other.probs)
        return as_tensor(p * torch.log(p / q) + (1.0 - p) * torch.log((1.0 - p) / (1.0 - q)))


Geometric = type("Geometric", (_GeometricMixin, Geometric), {})


def _bernoulli_cdf(self, value):
    """0 below 0, 1 - p on [0, 1), 1 from 1 on."""
    v, p = _t(value), _t(self.probs)
    v, p = torch.broadcast_tensors(v, p)
    return as_tensor(torch.where(v < 0, torch.zeros_like(p), torch.where(v < 1, 1 - p, torch.ones_like(p))))


Bernoulli.cdf = _bernoulli_cdf


def _poisson_entropy(self):
    """Sum of -p log p over the support up to rate + 30 sqrt(rate) (the tail beyond is below float precision)."""
    rate = _t(self.rate)
    hi = int(torch.ceil(rate.max() + 30 * torch.sqrt(rate.max())).item()) + 1
    values = torch.arange(hi, dtype=rate.dtype).reshape((-1,) + (1,) * rate.dim())
    lp = self._d.log_prob(values)
    return as_tensor(-(lp.exp() * lp).sum(0) * (rate != 0).to(rate.dtype))


Poisson.entropy = _poisson_entropy


class Categorical(Distribution):
    """``Categorical(logits)``: Paddle's argument is un-normalised NON-log weights when positive, as in
    categorical.py:94 (probabilities are ``logits / sum(logits)``)."""

    def __init__(self, logits, name=None):
        lg = _t(logits)
        self.logits = as_tensor(lg)
        self._d = D.Categorical(probs=lg / lg.sum(-1, keepdim=True))

    def probs(self, value):
        return as_tensor(self._d.probs.gather(-1, _t(value).long().unsqueeze(-1)).squeeze(-1)) \
            if self._d.probs.dim() > 1 else as_tensor(self._d.probs[_t(value).long()])


class Independent(Distribution):
    def __init__(self, base, reinterpreted_batch_rank):
        self._d = D.Independent(base._d, reinterpreted_batch_rank)


# ------------------------------------------------------------------ transforms
class Transform:
    _t = None

    def forward(self, x):
        return as_tensor(self._t(_t(x)))

    __call__ = forward

    def inverse(self, y):
        return as_tensor(self._t.inv(_t(y)))

    def forward_log_det_jacobian(self, x):
        x = _t(x)
        return as_tensor(self._t.log_abs_det_jacobian(x, self._t(x)))

    def inverse_log_det_jacobian(self, y):
        y = _t(y)
        return as_tensor(-self._t.log_abs_det_jacobian(self._t.inv(y), y))

    def forward_shape(self, shape):
        return tuple(self._t.forward_shape(tuple(shape)))

    def inverse_shape(self, shape):
        return tuple(self._t.inverse_shape(tuple(shape)))


def _tr(name, factory):
    def __init__(self, *a, **k):
        self._t = factory(*[_t(v) for v in a], **{kk: _t(v) for kk, v in k.items()})
    return type(name, (Transform,), {"__init__": __init__})


AbsTransform = _tr("AbsTransform", D.transforms.AbsTransform)
AffineTransform = _tr("AffineTransform", D.transforms.AffineTransform)
ExpTransform = _tr("ExpTransform", D.transforms.ExpTransform)
PowerTransform = _tr("PowerTransform", lambda power: D.transforms.PowerTransform(power))
SigmoidTransform = _tr("SigmoidTransform", D.transforms.SigmoidTransform)
SoftmaxTransform = _tr("SoftmaxTransform", D.transforms.SoftmaxTransform)
StickBreakingTransform = _tr("StickBreakingTransform", D.transforms.StickBreakingTransform)
TanhTransform = _tr("TanhTransform", D.transforms.TanhTransform)
ReshapeTransform = _tr("ReshapeTransform", lambda in_event_shape, out_event_shape: D.transforms.ReshapeTransform(
    tuple(in_event_shape), tuple(out_event_shape)))


class ChainTransform(Transform):
    def __init__(self, transforms):
        self._t = D.transforms.ComposeTransform([t._t for t in transforms])


class IndependentTransform(Transform):
    def __init__(self, base, reinterpreted_batch_rank):
        self._t = D.transforms.IndependentTransform(base._t, reinterpreted_batch_rank)


class StackTransform(Transform):
    def __init__(self, transforms, axis=0):
        self._t = D.transforms.StackTransform([t._t for t in transforms], axis)


class TransformedDistribution(Distribution):
    def __init__(self, base, transforms):
        self._d = D.TransformedDistribution(base._d, [t._t for t in transforms])


_KL = {}


def register_kl(cls_p, cls_q):
    def deco(fn):
        _KL[(cls_p, cls_q)] = fn
        return fn
    return deco


def kl_divergence(p, q):
    for (cp, cq), fn in _KL.items():
        if isinstance(p, cp) and isinstance(q, cq):
            return fn(p, q)
    return as_tensor(D.kl_divergence(p._d, q._d))


from .._core.submodule_alias import alias_submodules as _alias  # noqa: E402
_alias(__name__, ("bernoulli", "beta", "binomial", "categorical", "cauchy", "chi2", "continuous_bernoulli", "dirichlet", "distribution",
                  "exponential", "exponential_family", "gamma", "geometric", "gumbel", "independent", "kl", "laplace", "lkj_cholesky",
                  "lognormal", "multinomial", "multivariate_normal", "normal", "poisson", "student_t", "transform", "transformed_distribution",
                  "uniform", "variable"))
