"""Tape autograd: gradients of a small expression, numerical gradient check and a Jacobian."""
import _path  # noqa: F401
import torch

from rustorch_b200 import autograd

x = torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64, requires_grad=True)
w = torch.tensor([0.5, -1.0, 2.0], dtype=torch.float64, requires_grad=True)
y = ((x * w).tanh() + x.pow(2)).sum()
y.backward()
print("y =", float(y), "dy/dx =", x.grad.tolist(), "dy/dw =", w.grad.tolist())

f = lambda a: (a * w.detach()).tanh() + a.pow(2)       # noqa: E731
print("gradcheck:", autograd.gradcheck(lambda a: f(a).sum(), (x.detach().clone().requires_grad_(True),)))
print("jacobian diag:", torch.diagonal(autograd.jacobian(f, x.detach()).data).tolist())
