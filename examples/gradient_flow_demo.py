"""Where gradients go: hooks, retained intermediate gradients, detach, no_grad, and a vanishing-gradient check on a
deep sigmoid stack against the same stack with residual connections."""
import _path  # noqa: F401

import torch

import rustorch as rt
from rustorch_b200 import autograd, nn

x = rt.Variable(torch.tensor([1.0, 2.0, 3.0]), requires_grad=True)
h = (x * 2.0).retain_grad()
seen = []
h.register_hook(lambda g: seen.append(g.as_slice()))
y = (h * h).sum()
y.backward()
print("dy/dh (retained):", h.grad.as_slice(), " hook saw:", seen[0], " dy/dx:", x.grad.as_slice())
d = (x.detach() * 3.0).sum()
print("detached branch requires_grad:", bool(d.requires_grad))
with rt.no_grad():
    print("inside no_grad requires_grad:", bool((x * 2.0).requires_grad))


def first_layer_grad(residual: bool, depth: int = 20) -> float:
    torch.manual_seed(0)
    layers = [nn.Linear(16, 16) for _ in range(depth)]
    t = torch.randn(8, 16)
    for l in layers:
        t = t + torch.sigmoid(l(t)) if residual else torch.sigmoid(l(t))
    t.sum().backward()
    return float(layers[0].weight.grad.norm())


print("gradient norm at the first of 20 sigmoid layers: plain %.2e, with residuals %.2e" % (first_layer_grad(False), first_layer_grad(True)))
an = autograd.GradientFlowAnalyzer(vanishing=1e-6)
torch.manual_seed(0)
deep = nn.Sequential(*[m for _ in range(12) for m in (nn.Linear(8, 8), nn.Sigmoid())])
for _ in range(3):
    deep.zero_grad()
    deep(torch.randn(4, 8)).sum().backward()
    an.record(deep.named_parameters())
flagged = an.issues()
print("analyzer flags", len(flagged), "parameters, e.g.", dict(list(flagged.items())[:2]))
