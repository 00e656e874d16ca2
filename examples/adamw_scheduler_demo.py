"""AdamW with learning-rate schedules: the schedule each scheduler produces and a short run with warm-up + cosine."""
import _path  # noqa: F401

import torch

import rustorch as rt
from rustorch_b200 import optim as O


def trace(make, steps=10, metric=None, lr=0.1):
    opt = O.AdamW([torch.nn.Parameter(torch.zeros(1))], lr=lr)
    sched = make(opt)
    out = []
    for i in range(steps):
        out.append(round(float(opt.learning_rate), 4))
        sched.step_with_metric(metric[i]) if metric else sched.step()
    return out


print("StepLR(3, 0.5)       ", trace(lambda o: O.StepLR(o, 3, 0.5)))
print("ExponentialLR(0.8)   ", trace(lambda o: O.ExponentialLR(o, 0.8)))
print("CosineAnnealing(10)  ", trace(lambda o: O.CosineAnnealingLR(o, 10, 0.0)))
print("MultiStep([2, 6])    ", trace(lambda o: O.MultiStepLR(o, [2, 6], 0.1)))
print("Warmup(0.01 -> 0.1) ", trace(lambda o: O.WarmupScheduler(o, 0.1, 5), lr=0.01))
print("OneCycle(0.5, 10)    ", trace(lambda o: O.OneCycleLR(o, 0.5, 10)))
print("Polynomial(10, 2)    ", trace(lambda o: O.PolynomialLR(o, 10, 2.0)))
print("ReduceLROnPlateau    ", trace(lambda o: O.ReduceLROnPlateau(o, patience=1, factor=0.5), metric=[1.0, 0.9, 0.9, 0.9, 0.9, 0.8, 0.8, 0.8, 0.8, 0.8]))

rt.set_seed(0)
X, y = torch.randn(256, 10), torch.randn(256, 1)
model = rt.Sequential(rt.Linear(10, 32), rt.GELU(), rt.Linear(32, 1))
opt = O.AdamW.with_weight_decay(model.parameters(), 3e-4, 0.05)          # warm-up starts from this rate
warm, cos = O.WarmupScheduler(opt, 3e-3, 5), None
for epoch in range(30):
    opt.zero_grad()
    loss = rt.MSELoss()(model(X), y)
    loss.backward()
    opt.step()
    if epoch < 5:
        warm.step()
    else:
        cos = cos or O.CosineAnnealingLR(opt, 25, 1e-5)
        cos.step()
    if epoch % 10 == 9:
        print(f"epoch {epoch + 1:2d}  lr {float(opt.learning_rate):.5f}  loss {float(loss.detach()):.4f}")
