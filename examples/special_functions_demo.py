"""Special functions: gamma family, error functions, Bessel functions, a few identities checked numerically."""
import _path  # noqa: F401
import math

import torch

from rustorch_b200 import special as S

x = torch.tensor([0.5, 1.0, 2.5, 5.0], dtype=torch.float64)
print("gamma   ", [round(float(v), 5) for v in S.gamma(x)])
print("lgamma  ", [round(float(v), 5) for v in S.lgamma(x)])
print("digamma ", [round(float(v), 5) for v in S.digamma(x)])
print("gamma(0.5)^2 = pi:", abs(float(S.gamma(torch.tensor(0.5, dtype=torch.float64))) ** 2 - math.pi) < 1e-12)
print("beta(2, 3) = 1/12:", abs(float(S.beta(torch.tensor(2.0), torch.tensor(3.0))) - 1 / 12) < 1e-6)
e = torch.tensor([-1.0, 0.0, 0.5, 2.0], dtype=torch.float64)
print("erf     ", [round(float(v), 6) for v in S.erf(e)], " erf + erfc = 1:", bool(torch.allclose(S.erf(e) + S.erfc(e), torch.ones_like(e))))
p = torch.tensor([-0.9, 0.0, 0.3, 0.99], dtype=torch.float64)
print("erfinv round trip:", bool(torch.allclose(S.erf(S.erfinv(p)), p, atol=1e-10)))
z = torch.tensor([0.5, 1.0, 2.0, 10.0], dtype=torch.float64)
print("J0      ", [round(float(v), 6) for v in S.bessel_j(0, z)])
print("Y1      ", [round(float(v), 6) for v in S.bessel_y(1, z)])
print("I0, K0  ", [round(float(v), 6) for v in S.bessel_i(0, z[:2])], [round(float(v), 6) for v in S.bessel_k(0, z[:2])])
print("5! =", S.factorial(5), " C(10, 3) =", S.binomial_coefficient(10, 3), " H_10 = %.6f" % S.harmonic_number(10))
