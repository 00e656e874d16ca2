"""Complex scalars and complex tensors (reference: src/tensor/complex.rs tests, complex_impl/*)."""
import math

import pytest
import torch

import rustorch_b200 as rt
from rustorch_b200 import complex as C
from rustorch_b200.complex import Complex
from rustorch_b200.tensor import Tensor


def test_scalar_arithmetic_and_properties():
    z1, z2 = Complex.new(3.0, 4.0), Complex.new(1.0, 2.0)
    assert Complex.from_real(5.0) == Complex(5.0, 0.0) and Complex.from_imag(2.0) == Complex(0.0, 2.0)
    assert z1 + z2 == Complex(4.0, 6.0) and z1 - z2 == Complex(2.0, 2.0) and z1 * z2 == Complex(-5.0, 10.0)
    d = z1 / z2
    assert d.real() == pytest.approx(2.2, abs=1e-12) and d.imag() == pytest.approx(-0.4, abs=1e-12)
    assert z1.abs() == pytest.approx(5.0) and z1.abs_sq() == pytest.approx(25.0) and z1.conj() == Complex(3.0, -4.0)
    assert z1.arg() == pytest.approx(math.atan2(4.0, 3.0))
    r, th = z1.to_polar()
    back = Complex.from_polar(r, th)
    assert back.real() == pytest.approx(3.0) and back.imag() == pytest.approx(4.0)
    assert Complex.zero_const() == Complex(0, 0) and Complex.one_const() == Complex(1, 0) and Complex.i() == Complex(0, 1)
    assert z1.is_finite() and not z1.is_nan() and Complex(float("inf"), 0).is_infinite() and Complex(2, 0).is_real() and Complex(0, 2).is_imag()
    assert rt.Complex is Complex and 2 * z2 == Complex(2.0, 4.0) and (1 - z2) == Complex(0.0, -2.0)


def test_scalar_functions():
    z = Complex(1.0, 1.0)
    e = z.exp()
    assert e.real() == pytest.approx(math.e * math.cos(1.0)) and e.imag() == pytest.approx(math.e * math.sin(1.0))
    s = z.sqrt()
    assert (s * s).real() == pytest.approx(1.0) and (s * s).imag() == pytest.approx(1.0)
    w = Complex(0.5, 0.3)
    ident = w.sin() * w.sin() + w.cos() * w.cos()
    assert ident.real() == pytest.approx(1.0) and ident.imag() == pytest.approx(0.0, abs=1e-12)
    assert Complex.zero().pow(Complex.zero()) == Complex.one() and Complex.zero().pow(Complex(2, 0)) == Complex.zero()
    p = Complex(2.0, 0.0).pow(Complex(3.0, 0.0))
    assert p.real() == pytest.approx(8.0) and p.imag() == pytest.approx(0.0, abs=1e-12)
    ln = Complex(-1.0, 0.0).ln()
    assert ln.real() == pytest.approx(0.0, abs=1e-12) and ln.imag() == pytest.approx(math.pi)
    t = w.tanh()
    ref = complex(w.sinh()) / complex(w.cosh())
    assert complex(t) == pytest.approx(ref)


def test_tensor_construction_and_parts():
    real, imag = Tensor(torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64)), Tensor(torch.tensor([4.0, 5.0, 6.0], dtype=torch.float64))
    z = C.from_tensors(real, imag)
    assert z.data.dtype == torch.complex128 and tuple(z.data.shape) == (3,)
    assert C.tensor_real_part(z).data.tolist() == [1.0, 2.0, 3.0] and C.tensor_imag_part(z).data.tolist() == [4.0, 5.0, 6.0]
    torch.testing.assert_close(C.tensor_abs(z).data, torch.tensor([17.0, 29.0, 45.0], dtype=torch.float64).sqrt())
    assert C.tensor_conj(z).data.tolist() == [1 - 4j, 2 - 5j, 3 - 6j]
    assert z.real_part().data.tolist() == [1.0, 2.0, 3.0] and z.is_complex() and z.conj().data.tolist() == [1 - 4j, 2 - 5j, 3 - 6j]
    with pytest.raises(ValueError):
        C.from_tensors(torch.zeros(2), torch.zeros(3))
    assert (C.complex_zeros([2, 3]).data == 0).all() and (C.complex_ones([2, 2]).data == 1).all()
    assert (C.complex_i([1, 4]).data == 1j).all()
    p = C.from_polar(torch.tensor([1.0, 2.0], dtype=torch.float64), torch.tensor([0.0, math.pi / 2], dtype=torch.float64))
    torch.testing.assert_close(p.data, torch.tensor([1 + 0j, 2j], dtype=torch.complex128), atol=1e-12, rtol=0)
    assert C.from_real([1.0, 2.0]).data.tolist() == [1 + 0j, 2 + 0j] and C.from_imag([1.0]).data.tolist() == [1j]


def test_tensor_functions_match_scalar_definitions():
    g = torch.Generator().manual_seed(0)
    z = torch.complex(torch.randn(50, generator=g, dtype=torch.float64), torch.randn(50, generator=g, dtype=torch.float64))
    for name in ("exp", "sqrt", "sin", "cos", "tan", "sinh", "cosh", "tanh", "ln"):
        got = getattr(C, name)(z).data
        want = torch.tensor([complex(getattr(Complex._of(complex(v)), name)()) for v in z.tolist()], dtype=torch.complex128)
        torch.testing.assert_close(got, want, rtol=1e-9, atol=1e-9)
    w = torch.complex(torch.randn(50, generator=g, dtype=torch.float64), torch.randn(50, generator=g, dtype=torch.float64))
    z2 = z.clone()
    z2[0], w[0] = 0, 0
    z2[1] = 0
    got = C.pow(z2, w).data
    want = torch.tensor([complex(Complex._of(complex(a)).pow(complex(b))) for a, b in zip(z2.tolist(), w.tolist())], dtype=torch.complex128)
    torch.testing.assert_close(got, want, rtol=1e-9, atol=1e-9)
    assert got[0] == 1 and got[1] == 0
    torch.testing.assert_close(C.pow_scalar(z, 2.0).data, z * z, rtol=1e-9, atol=1e-9)


def test_matrix_ops():
    a = torch.tensor([[1 + 2j, 3 - 1j], [0.5j, 2.0 + 0j]], dtype=torch.complex128)
    b = torch.tensor([[2 - 1j, 1j], [1 + 1j, -1 + 0j]], dtype=torch.complex128)
    want = torch.zeros(2, 2, dtype=torch.complex128)
    for i in range(2):
        for j in range(2):
            want[i, j] = sum(a[i, k] * b[k, j] for k in range(2))
    torch.testing.assert_close(C.matmul(a, b).data, want)
    assert C.transpose(a).data[0, 1] == a[1, 0] and C.conj_transpose(a).data[0, 1] == a[1, 0].conj()
    assert complex(C.trace(a)) == complex(a[0, 0] + a[1, 1])
    assert complex(C.determinant(a)) == pytest.approx(complex(a[0, 0] * a[1, 1] - a[0, 1] * a[1, 0]))
    m3 = torch.randn(3, 3, dtype=torch.complex128)
    assert complex(C.determinant(m3)) == pytest.approx(complex(torch.linalg.det(m3)))
    with pytest.raises(ValueError):
        C.matmul(a, torch.zeros(3, 2, dtype=torch.complex128))
    with pytest.raises(ValueError):
        C.determinant(torch.zeros(2, 3, dtype=torch.complex128))


def test_fft_matches_dft_definition_and_normalisations():
    g = torch.Generator().manual_seed(1)
    for n in (8, 12, 1):
        x = torch.complex(torch.randn(n, generator=g, dtype=torch.float64), torch.randn(n, generator=g, dtype=torch.float64))
        k = torch.arange(n, dtype=torch.float64)
        dft = torch.exp(-2j * math.pi * k[:, None] * k[None, :] / n).to(torch.complex128)
        torch.testing.assert_close(C.fft(x).data, dft @ x, rtol=1e-9, atol=1e-9)
        torch.testing.assert_close(C.fft(x, norm="forward").data, dft @ x / n, rtol=1e-9, atol=1e-9)
        torch.testing.assert_close(C.fft(x, norm="ortho").data, dft @ x / math.sqrt(n), rtol=1e-9, atol=1e-9)
        torch.testing.assert_close(C.ifft(C.fft(x)).data, x, rtol=1e-9, atol=1e-9)
        torch.testing.assert_close(Tensor(x).fft(norm="ortho").ifft(norm="ortho").data, x, rtol=1e-9, atol=1e-9)
    with pytest.raises(ValueError):
        C.fft(torch.zeros(4), norm="bogus")
    x = torch.arange(5, dtype=torch.float64) + 0j
    assert C.fftshift(x).data.real.tolist() == [3.0, 4.0, 0.0, 1.0, 2.0]      # second half (from ceil(n/2)) first
    assert C.ifftshift(x).data.real.tolist() == [2.0, 3.0, 4.0, 0.0, 1.0]     # split at floor(n/2)
    torch.testing.assert_close(C.ifftshift(C.fftshift(x)).data, x)
    pad = C.fft(torch.ones(3, dtype=torch.float64), n=8).data
    assert pad.shape == (8,) and pad[0] == pytest.approx(3.0)
