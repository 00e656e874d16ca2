"""Probability distributions: ``Normal Uniform Bernoulli Categorical Exponential Gamma Beta`` with
``sample / rsample / log_prob / cdf / icdf / entropy / mean / variance``
(src/distributions/distribution.rs:29-140, normal.rs:50-80, gamma.rs:56-140, beta.rs, bernoulli.rs,
categorical.rs, exponential.rs, uniform.rs).

Sampling runs on the parameters' device with torch's Philox generator (the reference draws on the host
with Box–Muller / Marsaglia–Tsang loops).  ``rsample`` is reparameterised where the reference's is.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from ..special import lbeta


def _tt(x, like: Optional[torch.Tensor] = None) -> torch.Tensor:
    if isinstance(x, torch.Tensor):
        return x
    return torch.tensor(float(x), dtype=like.dtype if like is not None else torch.float32, device=like.device if like is not None else None)


class Distribution:
    """Base: batch/event shapes, argument validation, shape expansion (the ``DistributionTrait``)."""

    name = "distribution"

    def __init__(self, batch_shape: Sequence[int] = (), event_shape: Sequence[int] = (), validate_args: bool = True):
        self.batch_shape, self.event_shape, self.validate_args = tuple(batch_shape), tuple(event_shape), validate_args

    def expand_shape(self, sample_shape: Optional[Sequence[int]] = None) -> tuple:
        return tuple(sample_shape or ()) + self.batch_shape + self.event_shape

    def _check(self, cond: torch.Tensor, msg: str) -> None:
        if self.validate_args and not bool(cond.all()):
            raise ValueError(f"{self.name}: {msg}")

    def sample(self, sample_shape: Optional[Sequence[int]] = None, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        with torch.no_grad():
            return self.rsample(sample_shape, generator)

    def rsample(self, sample_shape=None, generator=None) -> torch.Tensor:
        raise NotImplementedError(f"{self.name} has no reparameterised sampler")

    def log_prob(self, value): raise NotImplementedError
    def cdf(self, value): raise NotImplementedError
    def icdf(self, value): raise NotImplementedError
    def entropy(self): raise NotImplementedError

    @property
    def stddev(self) -> torch.Tensor:
        return self.variance.sqrt()

    def prob(self, value) -> torch.Tensor:
        return self.log_prob(value).exp()


class Normal(Distribution):
    name = "Normal"

    def __init__(self, loc, scale, validate_args: bool = True):
        self.loc = _tt(loc)
        self.scale = _tt(scale, self.loc)
        self.loc, self.scale = torch.broadcast_tensors(self.loc, self.scale)
        super().__init__(self.loc.shape, (), validate_args)
        self._check(self.scale > 0, "scale must be positive")

    @classmethod
    def standard(cls, validate_args: bool = True) -> "Normal":
        return cls(0.0, 1.0, validate_args)

    from_scalars = classmethod(lambda cls, loc, scale, validate_args=True: cls(loc, scale, validate_args))

    def rsample(self, sample_shape=None, generator=None):
        eps = torch.randn(self.expand_shape(sample_shape), dtype=self.loc.dtype, device=self.loc.device, generator=generator)
        return self.loc + self.scale * eps

    def log_prob(self, value):
        z = (_tt(value, self.loc) - self.loc) / self.scale
        return -0.5 * z * z - self.scale.log() - 0.5 * math.log(2 * math.pi)

    def cdf(self, value):
        return 0.5 * (1 + torch.erf((_tt(value, self.loc) - self.loc) / (self.scale * math.sqrt(2))))

    def icdf(self, p):
        return self.loc + self.scale * math.sqrt(2) * torch.erfinv(2 * _tt(p, self.loc) - 1)

    def entropy(self):
        return 0.5 + 0.5 * math.log(2 * math.pi) + self.scale.log()

    mean = property(lambda self: self.loc)
    variance = property(lambda self: self.scale ** 2)


class Uniform(Distribution):
    name = "Uniform"

    def __init__(self, low, high, validate_args: bool = True):
        self.low = _tt(low)
        self.high = _tt(high, self.low)
        self.low, self.high = torch.broadcast_tensors(self.low, self.high)
        super().__init__(self.low.shape, (), validate_args)
        self._check(self.low < self.high, "low must be below high")

    def rsample(self, sample_shape=None, generator=None):
        u = torch.rand(self.expand_shape(sample_shape), dtype=self.low.dtype, device=self.low.device, generator=generator)
        return self.low + (self.high - self.low) * u

    def log_prob(self, value):
        v = _tt(value, self.low)
        inside = (v >= self.low) & (v < self.high)
        return torch.where(inside, -(self.high - self.low).log(), torch.full_like(v + self.low, -math.inf))

    def cdf(self, value):
        return ((_tt(value, self.low) - self.low) / (self.high - self.low)).clamp(0, 1)

    def icdf(self, p):
        return self.low + _tt(p, self.low) * (self.high - self.low)

    def entropy(self):
        return (self.high - self.low).log()

    mean = property(lambda self: (self.low + self.high) / 2)
    variance = property(lambda self: (self.high - self.low) ** 2 / 12)


class Bernoulli(Distribution):
    name = "Bernoulli"

    def __init__(self, probs=None, logits=None, validate_args: bool = True):
        if (probs is None) == (logits is None):
            raise ValueError("Bernoulli: give exactly one of probs / logits")
        if probs is not None:
            self.probs = _tt(probs)
            self.logits = torch.logit(self.probs.clamp(1e-12, 1 - 1e-12))
        else:
            self.logits = _tt(logits)
            self.probs = torch.sigmoid(self.logits)
        super().__init__(self.probs.shape, (), validate_args)
        self._check((self.probs >= 0) & (self.probs <= 1), "probs must lie in [0, 1]")

    def sample(self, sample_shape=None, generator=None):
        p = self.probs.expand(self.expand_shape(sample_shape))
        return torch.bernoulli(p, generator=generator)

    def log_prob(self, value):
        v = _tt(value, self.probs)
        return -torch.nn.functional.binary_cross_entropy_with_logits(self.logits.expand_as(v + self.logits), v.expand_as(v + self.logits), reduction="none")

    def cdf(self, value):
        v = _tt(value, self.probs)
        return torch.where(v < 0, torch.zeros_like(v + self.probs), torch.where(v < 1, 1 - self.probs + 0 * v, torch.ones_like(v + self.probs)))

    def entropy(self):
        return torch.nn.functional.binary_cross_entropy_with_logits(self.logits, self.probs, reduction="none")

    mean = property(lambda self: self.probs)
    variance = property(lambda self: self.probs * (1 - self.probs))


class Categorical(Distribution):
    name = "Categorical"

    def __init__(self, probs=None, logits=None, validate_args: bool = True):
        if (probs is None) == (logits is None):
            raise ValueError("Categorical: give exactly one of probs / logits")
        if probs is not None:
            p = _tt(probs)
            if validate_args and bool((p < 0).any()):
                raise ValueError("Categorical: probs must be non-negative")
            self.probs = p / p.sum(-1, keepdim=True)
            self.logits = self.probs.clamp_min(1e-38).log()
        else:
            self.logits = torch.log_softmax(_tt(logits), -1)
            self.probs = self.logits.exp()
        super().__init__(self.probs.shape[:-1], (), validate_args)
        self.num_categories = self.probs.shape[-1]

    def sample(self, sample_shape=None, generator=None):
        shape = tuple(sample_shape or ())
        n = max(1, math.prod(shape))
        flat = self.probs.reshape(-1, self.num_categories)
        idx = torch.multinomial(flat, n, replacement=True, generator=generator)       # [batch, n]
        return idx.t().reshape(shape + self.batch_shape)

    def log_prob(self, value):
        v = value.long()
        lg = self.logits.expand(v.shape + (self.num_categories,))
        return lg.gather(-1, v.unsqueeze(-1)).squeeze(-1)

    def entropy(self):
        return -(self.probs * self.logits).sum(-1)

    @property
    def mean(self):
        return (self.probs * torch.arange(self.num_categories, device=self.probs.device, dtype=self.probs.dtype)).sum(-1)

    @property
    def variance(self):
        k = torch.arange(self.num_categories, device=self.probs.device, dtype=self.probs.dtype)
        return (self.probs * k * k).sum(-1) - self.mean ** 2


class Exponential(Distribution):
    name = "Exponential"

    def __init__(self, rate, validate_args: bool = True):
        self.rate = _tt(rate)
        super().__init__(self.rate.shape, (), validate_args)
        self._check(self.rate > 0, "rate must be positive")

    def rsample(self, sample_shape=None, generator=None):
        u = torch.rand(self.expand_shape(sample_shape), dtype=self.rate.dtype, device=self.rate.device, generator=generator)
        return -torch.log1p(-u) / self.rate

    def log_prob(self, value):
        v = _tt(value, self.rate)
        return torch.where(v >= 0, self.rate.log() - self.rate * v, torch.full_like(v + self.rate, -math.inf))

    def cdf(self, value):
        return (1 - torch.exp(-self.rate * _tt(value, self.rate))).clamp_min(0)

    def icdf(self, p):
        return -torch.log1p(-_tt(p, self.rate)) / self.rate

    def entropy(self):
        return 1 - self.rate.log()

    mean = property(lambda self: 1 / self.rate)
    variance = property(lambda self: self.rate ** -2)


class Gamma(Distribution):
    name = "Gamma"

    def __init__(self, concentration, rate, validate_args: bool = True):
        self.concentration = _tt(concentration)
        self.rate = _tt(rate, self.concentration)
        self.concentration, self.rate = torch.broadcast_tensors(self.concentration, self.rate)
        super().__init__(self.rate.shape, (), validate_args)
        self._check((self.concentration > 0) & (self.rate > 0), "concentration and rate must be positive")

    from_concentration_rate = classmethod(lambda cls, c, r, validate_args=True: cls(c, r, validate_args))
    from_concentration_scale = classmethod(lambda cls, c, s, validate_args=True: cls(c, 1.0 / _tt(s), validate_args))
    exponential = classmethod(lambda cls, rate, validate_args=True: cls(1.0, rate, validate_args))

    def get_rate(self):
        return self.rate

    def get_scale(self):
        return 1 / self.rate

    def rsample(self, sample_shape=None, generator=None):
        c = self.concentration.expand(self.expand_shape(sample_shape))
        return torch._standard_gamma(c.contiguous()) / self.rate      # implicit reparameterisation gradients

    def log_prob(self, value):
        v = _tt(value, self.rate)
        return self.concentration * self.rate.log() + (self.concentration - 1) * v.log() - self.rate * v - torch.lgamma(self.concentration)

    def cdf(self, value):
        return torch.special.gammainc(self.concentration, self.rate * _tt(value, self.rate))

    def entropy(self):
        a = self.concentration
        return a - self.rate.log() + torch.lgamma(a) + (1 - a) * torch.digamma(a)

    mean = property(lambda self: self.concentration / self.rate)
    variance = property(lambda self: self.concentration / self.rate ** 2)


def betainc(a: torch.Tensor, b: torch.Tensor, x: torch.Tensor, iters: int = 200) -> torch.Tensor:
    """Regularised incomplete beta I_x(a, b): modified Lentz continued fraction, vectorised on the device."""
    a, b, x = torch.broadcast_tensors(a.double(), b.double(), x.double())
    swap = x > (a + 1) / (a + b + 2)
    aa, bb, xx = torch.where(swap, b, a), torch.where(swap, a, b), torch.where(swap, 1 - x, x)
    tiny = 1e-300
    c = torch.ones_like(xx)
    d = 1 - (aa + bb) * xx / (aa + 1)
    d = 1 / torch.where(d.abs() < tiny, torch.full_like(d, tiny), d)
    h = d.clone()
    for m in range(1, iters + 1):
        m2 = 2 * m
        num = m * (bb - m) * xx / ((aa + m2 - 1) * (aa + m2))
        d = 1 + num * d
        d = 1 / torch.where(d.abs() < tiny, torch.full_like(d, tiny), d)
        c = 1 + num / c
        c = torch.where(c.abs() < tiny, torch.full_like(c, tiny), c)
        h = h * d * c
        num = -(aa + m) * (aa + bb + m) * xx / ((aa + m2) * (aa + m2 + 1))
        d = 1 + num * d
        d = 1 / torch.where(d.abs() < tiny, torch.full_like(d, tiny), d)
        c = 1 + num / c
        c = torch.where(c.abs() < tiny, torch.full_like(c, tiny), c)
        delta = d * c
        h = h * delta
        if float((delta - 1).abs().max()) < 1e-14:
            break
    front = torch.exp(aa * xx.clamp_min(tiny).log() + bb * (1 - xx).clamp_min(tiny).log() - lbeta(aa, bb)) / aa
    res = front * h
    res = torch.where(swap, 1 - res, res)
    return torch.where(x <= 0, torch.zeros_like(res), torch.where(x >= 1, torch.ones_like(res), res))


class Beta(Distribution):
    name = "Beta"

    def __init__(self, concentration1, concentration0, validate_args: bool = True):
        self.alpha = _tt(concentration1)
        self.beta = _tt(concentration0, self.alpha)
        self.alpha, self.beta = torch.broadcast_tensors(self.alpha, self.beta)
        super().__init__(self.alpha.shape, (), validate_args)
        self._check((self.alpha > 0) & (self.beta > 0), "concentrations must be positive")

    def rsample(self, sample_shape=None, generator=None):
        shape = self.expand_shape(sample_shape)
        x = torch._standard_gamma(self.alpha.expand(shape).contiguous())
        y = torch._standard_gamma(self.beta.expand(shape).contiguous())
        return x / (x + y)

    def log_prob(self, value):
        v = _tt(value, self.alpha)
        return (self.alpha - 1) * v.log() + (self.beta - 1) * torch.log1p(-v) - lbeta(self.alpha, self.beta)

    def cdf(self, value):
        return betainc(self.alpha, self.beta, _tt(value, self.alpha)).to(self.alpha.dtype)

    def entropy(self):
        a, b = self.alpha, self.beta
        return lbeta(a, b) - (a - 1) * torch.digamma(a) - (b - 1) * torch.digamma(b) + (a + b - 2) * torch.digamma(a + b)

    mean = property(lambda self: self.alpha / (self.alpha + self.beta))
    variance = property(lambda self: self.alpha * self.beta / ((self.alpha + self.beta) ** 2 * (self.alpha + self.beta + 1)))


_REGISTRY = {"normal": Normal, "uniform": Uniform, "bernoulli": Bernoulli, "categorical": Categorical,
             "exponential": Exponential, "gamma": Gamma, "beta": Beta}


def available_distributions() -> list:
    return sorted(_REGISTRY)


def get_distribution(name: str):
    try:
        return _REGISTRY[name.lower()]
    except KeyError:
        raise ValueError(f"unknown distribution '{name}'; available: {available_distributions()}") from None
