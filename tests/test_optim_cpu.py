"""Optimizers, schedulers and utilities on CPU."""
import math

import pytest
import torch

from rustorch_b200 import optim


def _quad(opt_cls, steps=200, **kw):
    p = torch.nn.Parameter(torch.tensor([3.0, -2.0]))
    opt = opt_cls([p], **kw)
    for _ in range(steps):
        opt.zero_grad()
        (p * p).sum().backward()
        opt.step()
    return float(p.abs().max())


@pytest.mark.parametrize("cls,kw", [(optim.SGD, dict(lr=0.1, momentum=0.9)), (optim.Adam, dict(lr=0.1)),
                                    (optim.AdamW, dict(lr=0.1)), (optim.RMSprop, dict(lr=0.05)),
                                    (optim.AdaGrad, dict(lr=0.5)), (optim.NAdam, dict(lr=0.1)),
                                    (optim.RAdam, dict(lr=0.1)), (optim.Adamax, dict(lr=0.1)),
                                    (optim.AdaBound, dict(lr=0.1)), (optim.LAMB, dict(lr=0.05, weight_decay=0.0))])
def test_optimizers_minimise_quadratic(cls, kw):
    assert _quad(cls, **kw) < 0.1


def test_reference_defaults_and_api():
    p = [torch.nn.Parameter(torch.zeros(2))]
    a = optim.AdamW(p)
    g = a.param_groups[0]
    assert (g["betas"], g["eps"], g["weight_decay"], g["amsgrad"]) == ((0.9, 0.999), 1e-8, 0.01, False)
    assert optim.Adamax(p).param_groups[0]["eps"] == 1e-7
    assert optim.LAMB(p).param_groups[0]["eps"] == 1e-6 and optim.AdaGrad(p).param_groups[0]["eps"] == 1e-10
    assert optim.RMSprop.default_params(p).param_groups[0]["alpha"] == 0.99
    lb = optim.LBFGS(p).param_groups[0]
    assert (lb["max_iter"], lb["history_size"], lb["line_search_fn"]) == (20, 10, "strong_wolfe")
    s = optim.SGD.with_nesterov(p, 0.1, 0.9)
    assert s.param_groups[0]["nesterov"] and s.learning_rate() == 0.1
    s.set_lr(0.5)
    assert s.learning_rate() == 0.5
    assert "lr" in s.hyper_state()


def test_step_tensor_and_moments_in_state_dict():
    opt = optim.Adam(None, lr=0.1)
    w = torch.ones(3)
    opt.step_tensor(w, torch.ones(3))
    assert torch.allclose(w, torch.full((3,), 0.9), atol=1e-6)
    opt.step_tensor(w, torch.ones(3))           # second step on the same tensor: step count 2, not reset
    assert torch.allclose(w, torch.full((3,), 0.8), atol=1e-5)
    sd = opt.state_dict()
    assert any("exp_avg" in st for st in sd["state"].values())


def test_lbfgs_rosenbrock():
    p = torch.nn.Parameter(torch.tensor([-1.0, 1.5]))
    opt = optim.LBFGS([p], lr=1.0)

    def closure():
        opt.zero_grad()
        l = (1 - p[0]) ** 2 + 100 * (p[1] - p[0] ** 2) ** 2
        l.backward()
        return l

    for _ in range(10):
        opt.step(closure)
    assert torch.allclose(p.detach(), torch.ones(2), atol=1e-3)


def test_schedulers():
    p = [torch.nn.Parameter(torch.zeros(1))]
    o = optim.SGD(p, lr=1.0)
    s = optim.StepLR(o, 2, 0.5)
    assert [round(s.step(), 4) for _ in range(4)] == [1.0, 0.5, 0.5, 0.25]
    o = optim.SGD(p, lr=1.0)
    assert round(optim.ExponentialLR(o, 0.9).step(), 4) == 0.9
    o = optim.SGD(p, lr=1.0)
    c = optim.CosineAnnealingLR(o, 10, 0.0)
    lrs = [c.step() for _ in range(10)]
    assert abs(lrs[4] - 0.5) < 1e-6 and abs(lrs[-1]) < 1e-9
    o = optim.SGD(p, lr=1.0)
    assert [round(optim.MultiStepLR(o, [2, 3], 0.1).compute_lr(e), 4) for e in (1, 2, 3)] == [1.0, 0.1, 0.01]
    o = optim.SGD(p, lr=0.0)
    w = optim.WarmupScheduler(o, 1.0, 4)
    assert [w.step() for _ in range(5)] == [0.25, 0.5, 0.75, 1.0, 1.0]
    o = optim.SGD(p, lr=0.1)
    oc = optim.OneCycleLR(o, 1.0, 100, 0.3)
    lrs = [oc.step() for _ in range(100)]
    assert max(lrs) == pytest.approx(1.0) and lrs.index(max(lrs)) == 29 and lrs[-1] < 1e-4
    o = optim.SGD(p, lr=1.0)
    assert optim.PolynomialLR(o, 10, 2.0, 0.0).compute_lr(5) == pytest.approx(0.25)
    o = optim.SGD(p, lr=1.0)
    r = optim.ReduceLROnPlateau(o, optim.PlateauMode.MIN, 0.5, patience=1)
    for v in (1.0, 1.0, 1.0, 1.0):
        r.step_with_metric(v)
    assert o.learning_rate() == 0.5
    sd = r.state_dict()
    r.load_state_dict(sd)


def test_schedulers_drive_fused_optimizer():
    lin = torch.nn.Linear(4, 2)
    flat = optim.FlatParams(lin)
    fo = optim.FusedAdamW(flat, lr=1.0)
    s = optim.StepLR(fo, 1, 0.1)
    s.step()
    assert fo.learning_rate() == pytest.approx(0.1)


def test_utils():
    p = torch.nn.Parameter(torch.ones(4))
    p.grad = torch.full((4,), 10.0)
    assert optim.clip_grad_norm([p], 1.0) == pytest.approx(20.0)
    assert float(p.grad.norm()) == pytest.approx(1.0, rel=1e-4)
    p.grad = torch.tensor([float("nan"), 0, 0, 0])
    assert not optim.StabilityConfig().apply([p])
    m = optim.OptimizerMetrics(window=3, tolerance=1e-3)
    for v in (1.0, 0.5, 0.5, 0.5, 0.5):
        m.record(v)
    assert m.has_converged() and not m.is_diverging()
    assert optim.OptimizerFactory.suggest_parameters("transformer")["optimizer"] == "adamw"
    assert isinstance(optim.OptimizerFactory.create("radam", [p], lr=0.1), optim.RAdam)
    r = optim.OptimizerBenchmark(2, 100, 20).run("adamax")
    assert r["steps_per_s"] > 0
