"""Linear regression three ways: closed form, tape autograd with a hand-written update, and Linear + SGD."""
import _path  # noqa: F401

import torch

import rustorch as rt

rt.set_seed(0)
true_w, true_b = torch.tensor([2.0, -3.0, 0.5]), 1.5
X = torch.randn(200, 3)
y = X @ true_w + true_b + 0.05 * torch.randn(200)

A = torch.cat([X, torch.ones(200, 1)], 1)
sol = torch.linalg.lstsq(A, y.unsqueeze(1)).solution.flatten()
print("closed form      w =", [round(v, 3) for v in sol[:3].tolist()], " b = %.3f" % float(sol[3]))

w, b = rt.Variable.zeros([3], requires_grad=True), rt.Variable.zeros([1], requires_grad=True)
for _ in range(200):
    loss = ((rt.Variable(X).matmul(w) + b - rt.Variable(y)).pow(2.0)).mean()
    w.zero_grad(), b.zero_grad()
    loss.backward()
    with rt.no_grad():
        w.tensor -= 0.1 * w.grad.data
        b.tensor -= 0.1 * b.grad.data
print("Variable + manual w =", [round(v, 3) for v in w.tensor.tolist()], " b = %.3f  loss %.5f" % (float(b.tensor.detach()), float(loss.item())))

model = rt.Linear(3, 1)
opt = rt.SGD(model.parameters(), lr=0.1, momentum=0.9)
for _ in range(100):
    opt.zero_grad()
    out = rt.MSELoss()(model(X).squeeze(1), y)
    out.backward()
    opt.step()
print("Linear + SGD     w =", [round(v, 3) for v in model.weight.flatten().tolist()], " b = %.3f  loss %.5f" % (float(model.bias), float(out)))
