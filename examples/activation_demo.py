"""Activation layers and their functional forms; gradients of each at a few points."""
import _path  # noqa: F401

import torch

import rustorch as rt
from rustorch_b200 import nn

x = torch.linspace(-3, 3, 7)
layers = {"ReLU": nn.ReLU(), "LeakyReLU": nn.LeakyReLU(0.1), "Sigmoid": nn.Sigmoid(), "Tanh": nn.Tanh(), "GELU": nn.GELU(),
          "Swish": nn.Swish(), "ELU": nn.ELU(), "SELU": nn.SELU(), "Mish": nn.Mish(), "Softmax": nn.Softmax(-1)}
print("x        ", [f"{v:6.2f}" for v in x.tolist()])
for name, layer in layers.items():
    xv = x.clone().requires_grad_(True)
    y = layer(xv)
    y.sum().backward()
    print(f"{name:<9}", [f"{v:6.2f}" for v in y.tolist()], " d/dx at 0: %.3f" % float(xv.grad[3]))
v = rt.Variable(x, requires_grad=True)
print("functional on a Variable:", type(rt.gelu(v)).__name__, [round(a, 3) for a in rt.gelu(v).tensor.tolist()][:3])
glu = nn.GLU()
print("GLU halves the last dimension:", tuple(glu(torch.randn(2, 8)).shape))
