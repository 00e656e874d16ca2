"""Complex numbers and complex tensors: arithmetic, polar form, matrix product, FFT."""
import _path  # noqa: F401
import math

import torch

from rustorch_b200 import complex as C

a, b = C.Complex(3.0, 4.0), C.Complex.from_polar(2.0, math.pi / 2)
print("a =", a, "|a| =", abs(a), " b =", b)
print("a * b =", a * b, " a / b =", a / b, " conj(a) =", a.conj())
print("exp(i pi) =", C.Complex(0.0, math.pi).exp(), " sqrt(-4) =", C.Complex(-4.0, 0.0).sqrt(), " i^2 =", C.Complex(0.0, 1.0).pow(2))
m = C.from_tensors(torch.tensor([[1.0, 0.0], [0.0, 1.0]]), torch.tensor([[0.0, 1.0], [-1.0, 0.0]]))      # I + i J
print("matrix:", m.tolist())
print("m @ m^H:", C.matmul(m, C.conj_transpose(m)).tolist(), " det:", C.determinant(m))
sig = C.from_real(torch.sin(2 * math.pi * 4 * torch.arange(32) / 32))
spec = C.tensor_abs(C.fft(sig))
print("FFT of a 4-cycle sine peaks at bins", sorted(torch.topk(spec, 2).indices.tolist()))
print("ifft(fft(x)) == x:", bool(torch.allclose(C.tensor_real_part(C.ifft(C.fft(sig))), C.tensor_real_part(sig), atol=1e-5)))
