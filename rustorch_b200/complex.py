"""Complex numbers and complex tensors.

The reference has a ``Complex<T>`` scalar (src/tensor/complex_impl/core.rs:21-140, arithmetic.rs, math.rs:301-381)
and ``Tensor<Complex<T>>`` helpers: construction from real / imaginary or magnitude / phase tensors, part
extraction, element-wise transcendental functions (tensor_ops.rs:13-208) and matrix operations: matmul, transpose,
conjugate transpose, trace, determinant (1x1 and 2x2 only there), radix-2 FFT / inverse FFT with ``forward`` /
``backward`` / ``ortho`` normalisation and 1-D fftshift / ifftshift (matrix.rs:13-270).

Here a complex tensor is a ``torch.complex64 / complex128`` tensor (on the CPU or on the GPU, where the products and
the FFT run on the device), wrapped in the framework's :class:`~rustorch_b200.tensor.Tensor`.  The method names and
argument order are the reference's; the determinant works for any square matrix (LU), the FFT for any length and
along any dimension, and the shifts for any rank.  Branch cuts follow the reference: ``ln`` returns
``(ln|z|, arg z)`` with ``arg`` in ``(-pi, pi]``, ``sqrt`` halves the argument, ``pow`` is ``exp(w ln z)`` with
``0 ** 0 = 1`` and ``0 ** w = 0``.
"""
from __future__ import annotations

import cmath
import math
from typing import Optional, Sequence, Tuple, Union

import torch

from .tensor import Tensor, _unwrap

Real = Union[int, float]


class Complex:
    """One complex number with the reference's accessor and function names."""

    __slots__ = ("re", "im")

    def __init__(self, re: Real = 0.0, im: Real = 0.0):
        self.re, self.im = float(re), float(im)

    # ---- constructors / constants
    new = classmethod(lambda cls, re, im: cls(re, im))
    from_real = classmethod(lambda cls, re: cls(re, 0.0))
    from_imag = classmethod(lambda cls, im: cls(0.0, im))
    zero = zero_const = classmethod(lambda cls: cls(0.0, 0.0))
    one = one_const = classmethod(lambda cls: cls(1.0, 0.0))
    i = classmethod(lambda cls: cls(0.0, 1.0))

    @classmethod
    def from_polar(cls, r: Real, theta: Real) -> "Complex":
        return cls(r * math.cos(theta), r * math.sin(theta))

    @classmethod
    def _of(cls, z) -> "Complex":
        if isinstance(z, Complex):
            return z
        z = complex(z)
        return cls(z.real, z.imag)

    def __complex__(self) -> complex:
        return complex(self.re, self.im)

    # ---- parts and predicates
    def real(self) -> float:
        return self.re

    def imag(self) -> float:
        return self.im

    def conj(self) -> "Complex":
        return Complex(self.re, -self.im)

    def abs(self) -> float:
        return math.hypot(self.re, self.im)

    __abs__ = abs

    def abs_sq(self) -> float:
        return self.re * self.re + self.im * self.im

    def arg(self) -> float:
        return math.atan2(self.im, self.re)

    def to_polar(self) -> Tuple[float, float]:
        return self.abs(), self.arg()

    def is_finite(self) -> bool:
        return math.isfinite(self.re) and math.isfinite(self.im)

    def is_infinite(self) -> bool:
        return math.isinf(self.re) or math.isinf(self.im)

    def is_nan(self) -> bool:
        return math.isnan(self.re) or math.isnan(self.im)

    def is_real(self) -> bool:
        return self.im == 0.0

    def is_imag(self) -> bool:
        return self.re == 0.0

    def is_zero(self) -> bool:
        return self.re == 0.0 and self.im == 0.0

    # ---- arithmetic
    def __add__(self, o):
        o = Complex._of(o)
        return Complex(self.re + o.re, self.im + o.im)

    __radd__ = __add__

    def __sub__(self, o):
        o = Complex._of(o)
        return Complex(self.re - o.re, self.im - o.im)

    def __rsub__(self, o):
        return Complex._of(o) - self

    def __mul__(self, o):
        o = Complex._of(o)
        return Complex(self.re * o.re - self.im * o.im, self.re * o.im + self.im * o.re)

    __rmul__ = __mul__

    def __truediv__(self, o):
        o = Complex._of(o)
        d = o.abs_sq()
        return Complex((self.re * o.re + self.im * o.im) / d, (self.im * o.re - self.re * o.im) / d)

    def __rtruediv__(self, o):
        return Complex._of(o) / self

    def __neg__(self):
        return Complex(-self.re, -self.im)

    def __eq__(self, o) -> bool:
        try:
            o = Complex._of(o)
        except (TypeError, ValueError):
            return NotImplemented
        return self.re == o.re and self.im == o.im

    def __hash__(self):
        return hash((self.re, self.im))

    def __repr__(self) -> str:
        return f"Complex({self.re}, {self.im})"

    # ---- functions
    def exp(self) -> "Complex":
        e = math.exp(self.re)
        return Complex(e * math.cos(self.im), e * math.sin(self.im))

    def ln(self) -> "Complex":
        return Complex(math.log(self.abs()), self.arg())

    def pow(self, w) -> "Complex":
        w = Complex._of(w)
        if self.is_zero():
            return Complex.one() if w.is_zero() else Complex.zero()
        return (self.ln() * w).exp()

    __pow__ = pow

    def sqrt(self) -> "Complex":
        return Complex.from_polar(math.sqrt(self.abs()), self.arg() / 2.0)

    def _via(self, fn) -> "Complex":
        return Complex._of(fn(complex(self)))

    def sin(self):
        return self._via(cmath.sin)

    def cos(self):
        return self._via(cmath.cos)

    def tan(self):
        return self.sin() / self.cos()

    def sinh(self):
        return self._via(cmath.sinh)

    def cosh(self):
        return self._via(cmath.cosh)

    def tanh(self):
        return self.sinh() / self.cosh()


# ------------------------------------------------------------------------------------------ complex tensors
def _t(x) -> torch.Tensor:
    x = _unwrap(x)
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def _c(x) -> torch.Tensor:
    t = _t(x)
    if not t.is_complex():
        t = t.to(torch.complex128 if t.dtype == torch.float64 else torch.complex64)
    return t


def _cdtype(dtype) -> torch.dtype:
    if dtype in (torch.complex64, torch.complex128):
        return dtype
    return torch.complex128 if dtype in (torch.float64, None) else torch.complex64


def from_tensors(real, imag) -> Tensor:
    """Complex tensor from equally shaped real and imaginary parts (tensor_ops.rs:13-26)."""
    r, i = _t(real), _t(imag)
    if r.shape != i.shape:
        raise ValueError(f"real and imaginary parts must have the same shape, got {tuple(r.shape)} and {tuple(i.shape)}")
    if not r.is_floating_point():
        r, i = r.float(), i.float()
    return Tensor(torch.complex(r, i.to(r.dtype)))


def from_polar(magnitude, phase) -> Tensor:
    m, p = _t(magnitude), _t(phase)
    if m.shape != p.shape:
        raise ValueError("magnitude and phase must have the same shape")
    if not m.is_floating_point():
        m, p = m.float(), p.float()
    return Tensor(torch.polar(m, p.to(m.dtype)))


def from_real(real) -> Tensor:
    r = _t(real)
    return from_tensors(r, torch.zeros_like(r))


def from_imag(imag) -> Tensor:
    i = _t(imag)
    return from_tensors(torch.zeros_like(i), i)


def complex_zeros(shape: Sequence[int], dtype=torch.complex128, device=None) -> Tensor:
    return Tensor(torch.zeros(tuple(shape), dtype=_cdtype(dtype), device=device))


def complex_ones(shape: Sequence[int], dtype=torch.complex128, device=None) -> Tensor:
    return Tensor(torch.ones(tuple(shape), dtype=_cdtype(dtype), device=device))


def complex_i(shape: Sequence[int], dtype=torch.complex128, device=None) -> Tensor:
    return Tensor(torch.full(tuple(shape), 1j, dtype=_cdtype(dtype), device=device))


def tensor_real_part(z) -> Tensor:
    return Tensor(_c(z).real.clone())


def tensor_imag_part(z) -> Tensor:
    return Tensor(_c(z).imag.clone())


def tensor_abs(z) -> Tensor:
    return Tensor(_c(z).abs())


def tensor_arg(z) -> Tensor:
    return Tensor(_c(z).angle())


def tensor_conj(z) -> Tensor:
    return Tensor(_c(z).conj().resolve_conj())


def exp(z) -> Tensor:
    return Tensor(torch.exp(_c(z)))


def ln(z) -> Tensor:
    z = _c(z)
    return Tensor(torch.complex(z.abs().log(), z.angle()))


def pow(z, w) -> Tensor:  # noqa: A001  (reference name)
    """Element-wise ``z ** w`` = ``exp(w ln z)``; ``0 ** 0 = 1`` and ``0 ** w = 0`` (math.rs:314-326)."""
    z = _c(z)
    w = _c(w) if not isinstance(w, (int, float, complex, Complex)) else torch.full_like(z, complex(w))
    if w.shape != z.shape:
        w = w.expand_as(z)
    zero = z == 0
    safe = torch.where(zero, torch.ones_like(z), z)
    out = torch.exp(w * torch.complex(safe.abs().log(), safe.angle()))
    out = torch.where(zero, torch.where(w == 0, torch.ones_like(z), torch.zeros_like(z)), out)
    return Tensor(out)


def pow_scalar(z, w) -> Tensor:
    return pow(z, w)


def sqrt(z) -> Tensor:
    z = _c(z)
    return Tensor(torch.polar(z.abs().sqrt(), z.angle() / 2))


def sin(z) -> Tensor:
    return Tensor(torch.sin(_c(z)))


def cos(z) -> Tensor:
    return Tensor(torch.cos(_c(z)))


def tan(z) -> Tensor:
    return Tensor(torch.tan(_c(z)))


def sinh(z) -> Tensor:
    return Tensor(torch.sinh(_c(z)))


def cosh(z) -> Tensor:
    return Tensor(torch.cosh(_c(z)))


def tanh(z) -> Tensor:
    return Tensor(torch.tanh(_c(z)))


# ---- matrix operations (matrix.rs:13-152)
def matmul(a, b) -> Tensor:
    a, b = _c(a), _c(b)
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("complex matmul requires 2-D matrices")
    if a.shape[1] != b.shape[0]:
        raise ValueError(f"matrix dimensions do not match for multiplication: {tuple(a.shape)} x {tuple(b.shape)}")
    return Tensor(a @ b.to(a.dtype))


def transpose(z) -> Tensor:
    z = _c(z)
    if z.dim() != 2:
        raise ValueError("transpose requires a 2-D matrix")
    return Tensor(z.t().contiguous())


def conj_transpose(z) -> Tensor:
    z = _c(z)
    if z.dim() != 2:
        raise ValueError("conjugate transpose requires a 2-D matrix")
    return Tensor(z.t().conj().resolve_conj().contiguous())


def trace(z) -> Complex:
    z = _c(z)
    if z.dim() != 2:
        raise ValueError("trace requires a 2-D matrix")
    return Complex._of(complex(torch.diagonal(z).sum().item()))


def determinant(z) -> Complex:
    z = _c(z)
    if z.dim() != 2:
        raise ValueError("determinant requires a 2-D matrix")
    if z.shape[0] != z.shape[1]:
        raise ValueError("determinant requires a square matrix")
    return Complex._of(complex(torch.linalg.det(z).item()))


# ---- Fourier transforms (matrix.rs:154-270)
def _norm(norm: Optional[str]) -> str:
    norm = norm or "backward"
    if norm not in ("forward", "backward", "ortho"):
        raise ValueError(f"invalid normalization mode: {norm}")
    return norm


def fft(z, n: Optional[int] = None, dim: Optional[int] = None, norm: Optional[str] = None) -> Tensor:
    """Forward FFT: ``backward`` (default) leaves it unscaled, ``forward`` divides by n, ``ortho`` by sqrt(n)."""
    return Tensor(torch.fft.fft(_c(z), n=n, dim=-1 if dim is None else dim, norm=_norm(norm)))


def ifft(z, n: Optional[int] = None, dim: Optional[int] = None, norm: Optional[str] = None) -> Tensor:
    return Tensor(torch.fft.ifft(_c(z), n=n, dim=-1 if dim is None else dim, norm=_norm(norm)))


def fftshift(z, dim=None) -> Tensor:
    return Tensor(torch.fft.fftshift(_c(z), dim=dim))


def ifftshift(z, dim=None) -> Tensor:
    return Tensor(torch.fft.ifftshift(_c(z), dim=dim))


__all__ = ["Complex", "from_tensors", "from_polar", "from_real", "from_imag", "complex_zeros", "complex_ones", "complex_i",
           "tensor_real_part", "tensor_imag_part", "tensor_abs", "tensor_arg", "tensor_conj", "exp", "ln", "pow", "pow_scalar",
           "sqrt", "sin", "cos", "tan", "sinh", "cosh", "tanh", "matmul", "transpose", "conj_transpose", "trace", "determinant",
           "fft", "ifft", "fftshift", "ifftshift"]
