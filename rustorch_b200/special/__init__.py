"""Special functions on tensors: gamma family, error-function family, Bessel J/Y/I/K of integer order, and the
scalar helpers (src/special/gamma.rs:23-240, error.rs:22-365, bessel.rs:12-640, utils.rs:7-160).

Orders 0 and 1 use the device kernels behind ``torch.special``; higher integer orders use the standard
three-term recurrences (upward for Y and K, Miller's downward for J and I, which is the stable direction).
Everything is elementwise and runs on the tensor's device.
"""
from __future__ import annotations

import math
from typing import Union

import torch

TensorLike = Union[torch.Tensor, float]


def _t(x: TensorLike) -> torch.Tensor:
    return x if isinstance(x, torch.Tensor) else torch.tensor(float(x), dtype=torch.float64)


# ------------------------------------------------------------------ gamma family
def lgamma(x: TensorLike) -> torch.Tensor:
    return torch.lgamma(_t(x))


def gamma(x: TensorLike) -> torch.Tensor:
    """Gamma function with the sign of the reflection for negative non-integers; poles give ``inf``."""
    x = _t(x)
    mag = torch.exp(torch.lgamma(x))
    neg = x < 0
    sign = torch.where(neg & (torch.floor(x).to(torch.int64) % 2 != 0), -torch.ones_like(x), torch.ones_like(x))
    return mag * sign


def digamma(x: TensorLike) -> torch.Tensor:
    return torch.digamma(_t(x))


def polygamma(n: int, x: TensorLike) -> torch.Tensor:
    return torch.polygamma(n, _t(x))


def lbeta(a: TensorLike, b: TensorLike) -> torch.Tensor:
    a, b = _t(a), _t(b)
    return torch.lgamma(a) + torch.lgamma(b) - torch.lgamma(a + b)


def beta(a: TensorLike, b: TensorLike) -> torch.Tensor:
    return torch.exp(lbeta(a, b))


# ------------------------------------------------------------------ error functions
def erf(x: TensorLike) -> torch.Tensor:
    return torch.erf(_t(x))


def erfc(x: TensorLike) -> torch.Tensor:
    return torch.erfc(_t(x))


def erfinv(x: TensorLike) -> torch.Tensor:
    x = _t(x)
    if bool(((x < -1) | (x > 1)).any()):
        raise ValueError("erfinv: argument outside [-1, 1]")
    return torch.erfinv(x)


def erfcinv(x: TensorLike) -> torch.Tensor:
    x = _t(x)
    if bool(((x < 0) | (x > 2)).any()):
        raise ValueError("erfcinv: argument outside [0, 2]")
    return torch.erfinv(1.0 - x)


def erfcx(x: TensorLike) -> torch.Tensor:
    """Scaled complementary error function ``exp(x^2) erfc(x)``."""
    return torch.special.erfcx(_t(x))


# ------------------------------------------------------------------ Bessel functions
def _int_order(n) -> int:
    if float(n) != int(n):
        raise ValueError("only integer orders are supported")
    return int(n)


def _miller(n: int, x: torch.Tensor, modified: bool) -> torch.Tensor:
    """Downward recurrence from a start order well above ``n``, normalised with the order-0 value."""
    f0 = torch.special.i0(x) if modified else torch.special.bessel_j0(x)
    ax = x.abs().clamp_min(1e-30)
    start = 2 * ((n + int(math.sqrt(40.0 * n)) + int(float(ax.max())) + 8) // 2)
    bkp, bk = torch.zeros_like(x), torch.full_like(x, 1e-30)
    out = torch.zeros_like(x)
    for k in range(start, 0, -1):
        bkm = (2.0 * k / ax) * bk + bkp if modified else (2.0 * k / ax) * bk - bkp
        bkp, bk = bk, bkm
        big = bk.abs() > 1e100                              # rescale to stay in range
        scale = torch.where(big, torch.full_like(x, 1e-100), torch.ones_like(x))
        bk, bkp, out = bk * scale, bkp * scale, out * scale
        if k - 1 == n:
            out = bk.clone()
    res = out * (f0 / bk)
    if n % 2:
        res = torch.where(x < 0, -res, res)
    return torch.where(x == 0, torch.zeros_like(x) if n > 0 else torch.ones_like(x), res)


def bessel_j(n, x: TensorLike) -> torch.Tensor:
    n, x = _int_order(n), _t(x)
    if n < 0:
        return (-1) ** n * bessel_j(-n, x)
    if n == 0:
        return torch.special.bessel_j0(x)
    if n == 1:
        return torch.special.bessel_j1(x)
    # upward recurrence is stable while |x| > n; Miller's algorithm otherwise
    return torch.where(x.abs() > n, _upward_j(n, x), _miller(n, x, modified=False))


def _upward_j(n: int, x: torch.Tensor) -> torch.Tensor:
    ax = x.abs().clamp_min(1e-30)
    a, b = torch.special.bessel_j0(ax), torch.special.bessel_j1(ax)
    for k in range(1, n):
        a, b = b, (2.0 * k / ax) * b - a
    return torch.where((x < 0) & (n % 2 == 1), -b, b)


def bessel_y(n, x: TensorLike) -> torch.Tensor:
    n, x = _int_order(n), _t(x)
    if bool((x <= 0).any()):
        raise ValueError("bessel_y: x must be positive")
    if n < 0:
        return (-1) ** n * bessel_y(-n, x)
    a = torch.special.bessel_y0(x)
    if n == 0:
        return a
    b = torch.special.bessel_y1(x)
    for k in range(1, n):
        a, b = b, (2.0 * k / x) * b - a
    return b


def bessel_i(n, x: TensorLike) -> torch.Tensor:
    n, x = abs(_int_order(n)), _t(x)
    if n == 0:
        return torch.special.i0(x)
    if n == 1:
        return torch.special.i1(x)
    return _miller(n, x, modified=True)


def bessel_k(n, x: TensorLike) -> torch.Tensor:
    n, x = abs(_int_order(n)), _t(x)
    if bool((x <= 0).any()):
        raise ValueError("bessel_k: x must be positive")
    a = torch.special.modified_bessel_k0(x)
    if n == 0:
        return a
    b = torch.special.modified_bessel_k1(x)
    for k in range(1, n):
        a, b = b, (2.0 * k / x) * b + a
    return b


# ------------------------------------------------------------------ scalar helpers
def factorial(n: int) -> float:
    return float(math.factorial(n)) if n <= 170 else math.inf


def double_factorial(n: int) -> float:
    r = 1.0
    while n > 1:
        r *= n
        n -= 2
    return r


def binomial_coefficient(n: int, k: int) -> float:
    return float(math.comb(n, k)) if 0 <= k <= n else 0.0


def pochhammer(x: float, n: int) -> float:
    r = 1.0
    for i in range(n):
        r *= x + i
    return r


def harmonic_number(n: int) -> float:
    return sum(1.0 / k for k in range(1, n + 1))


def bernoulli_number(n: int) -> float:
    """B_n with B_1 = -1/2 (Akiyama–Tanigawa in exact rationals)."""
    from fractions import Fraction
    if n == 1:
        return -0.5
    if n % 2 and n > 1:
        return 0.0
    a = [Fraction(0)] * (n + 1)
    for m in range(n + 1):
        a[m] = Fraction(1, m + 1)
        for j in range(m, 0, -1):
            a[j - 1] = j * (a[j - 1] - a[j])
    return float(a[0])


def is_integer(x: float, tolerance: float = 1e-10) -> bool:
    return abs(x - round(x)) < tolerance


def signum(x: float) -> float:
    return 0.0 if x == 0 else math.copysign(1.0, x)
