"""The first steps of the reference's README, through ``import rustorch``: tensors, arithmetic, autograd, a small
network, one optimisation loop."""
import _path  # noqa: F401

import rustorch as rt

a = rt.tensor([1.0, 2.0, 3.0, 4.0], [2, 2])
b = rt.tensor([5.0, 6.0, 7.0, 8.0], [2, 2])
print("a + b =", (a + b).as_slice(), " a * b =", (a * b).as_slice(), " a @ b =", a.matmul(b).as_slice())
print("a^T   =", a.transpose().as_slice(), " sum =", float(a.sum()), " mean =", float(a.mean()), " shape =", a.shape)

x = rt.Variable(rt.tensor([2.0, 3.0]), requires_grad=True)
y = (x * x + x * 3.0).sum()
y.backward()
print("d/dx (x^2 + 3x) at [2, 3] =", x.grad.as_slice())

rt.set_seed(0)
model = rt.Sequential(rt.Linear(2, 16), rt.ReLU(), rt.Linear(16, 1))
opt = rt.Adam(model.parameters(), lr=0.02)
inputs = rt.tensor([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]])
targets = rt.tensor([[0.0], [1.0], [1.0], [0.0]])
for step in range(300):
    opt.zero_grad()
    loss = rt.MSELoss()(model(inputs), targets)
    loss.backward()
    opt.step()
print(f"XOR after 300 steps: loss {loss:.5f}, outputs", [round(v, 2) for v in model(inputs).as_slice()])
