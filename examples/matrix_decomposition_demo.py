"""SVD, QR, LU, eigen-decompositions and what each reconstructs (the reference's svd / eigenvalue / matrix
decomposition demos in one program)."""
import _path  # noqa: F401

import torch

import rustorch as rt

torch.manual_seed(0)
a = rt.Tensor(torch.randn(5, 3))
u, s, v = a.svd()
print("SVD: singular values", [round(x, 4) for x in s.as_slice()],
      " |A - U S V^T| = %.2e" % float((a.data - u.data @ torch.diag(s.data) @ v.data.T).abs().max()))
rank1 = s.data[0] * torch.outer(u.data[:, 0], v.data[:, 0])
print("best rank-1 approximation error (spectral) = second singular value: %.4f vs %.4f"
      % (float(torch.linalg.matrix_norm(a.data - rank1, 2)), float(s.data[1])))
q, r = a.qr()
print("QR: Q^T Q = I: %s, R upper triangular: %s" % (bool(torch.allclose(q.data.T @ q.data, torch.eye(3), atol=1e-5)),
                                                       bool(torch.allclose(r.data, r.data.triu()))))
sq = rt.Tensor(torch.randn(4, 4))
l, up, p = sq.lu()
print("LU: |P L U - A| = %.2e" % float((p.data @ l.data @ up.data - sq.data).abs().max()))
sym = rt.Tensor(sq.data + sq.data.T)
w, vec = sym.symeig()
print("symmetric eigenvalues", [round(x, 4) for x in w.as_slice()],
      " |A v - w v| = %.2e" % float((sym.data @ vec.data - vec.data * w.data).abs().max()))
ew, _ = sq.eig()
print("general eigenvalues (complex):", [complex(round(z.real, 3), round(z.imag, 3)) for z in ew.data.tolist()])
spd = rt.Tensor(sq.data @ sq.data.T + 4 * torch.eye(4))
ch = spd.cholesky()
print("Cholesky: |L L^T - A| = %.2e, det = %.3f, |A A^-1 - I| = %.2e"
      % (float((ch.data @ ch.data.T - spd.data).abs().max()), float(torch.linalg.det(spd.data)),
         float((spd.data @ spd.inverse().data - torch.eye(4)).abs().max())))
