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


def test_named_constructors_of_the_rust_api():
    """``Type::new / default_params / with_*`` (src/optim/mod.rs:93-137,233-296,424-500; adamw.rs:39-80; nadam.rs:135-175;
    radam.rs:187-225; adamax.rs:133-171; lamb.rs:34-75; adabound.rs:35-70; lbfgs.rs:192-250), parameters first."""
    import rustorch_b200.optim as O
    p = lambda: [torch.nn.Parameter(torch.ones(3))]   # noqa: E731
    assert O.SGD.new(p(), 0.1).learning_rate == pytest.approx(0.1) and O.Adam.new(p(), 0.01, (0.8, 0.9), 1e-6).beta1 == pytest.approx(0.8)
    assert O.AdamW.with_weight_decay(p(), 1e-3, 0.1).weight_decay == pytest.approx(0.1) and O.AdamW.with_amsgrad(p(), 1e-3).amsgrad
    r = O.RMSprop.with_momentum(p(), 0.01, 0.9, 1e-7, 0.5)
    assert (r.param_groups[0]["alpha"], r.eps, r.momentum) == (0.9, pytest.approx(1e-7), pytest.approx(0.5))
    assert O.RMSprop.with_weight_decay(p(), 0.01, 0.99, 1e-8, 0.1).weight_decay == pytest.approx(0.1)
    assert O.AdaGrad.with_weight_decay(p(), 0.01, 1e-9, 0.2).eps == pytest.approx(1e-9)
    n = O.NAdam.with_momentum_decay(p(), 2e-3, 0.01)
    assert n.param_groups[0]["momentum_decay"] == 0.01 and O.NAdam.default_params(p()).learning_rate == pytest.approx(2e-3)
    assert O.NAdam.with_weight_decay(p(), 2e-3, 0.1).weight_decay == pytest.approx(0.1)
    assert O.Adamax.with_infinity_eps(p(), 2e-3, 1e-5).eps == pytest.approx(1e-5) and O.Adamax.default_params(p()).eps == pytest.approx(1e-7)
    assert O.Adamax.with_weight_decay(p(), 2e-3, 0.1).weight_decay == pytest.approx(0.1)
    la = O.LAMB.with_params(p(), 1e-3, 0.8, 0.9, 1e-5, 0.0)
    assert (la.beta1, la.beta2, la.eps, la.weight_decay) == tuple(pytest.approx(v) for v in (0.8, 0.9, 1e-5, 0.0))
    assert la.param_groups[0]["bias_correction"] and not O.LAMB.without_bias_correction(p(), 1e-3).param_groups[0]["bias_correction"]
    ab = O.AdaBound.with_params(p(), 1e-3, 0.05, gamma=1e-2)
    ab.set_final_lr(0.2)
    assert ab.param_groups[0]["final_lr"] == 0.2 and ab.param_groups[0]["gamma"] == 1e-2
    lb = O.LBFGS.with_params(p(), 0.5, 10, 15, 1e-6, 1e-10, 5, "StrongWolfe")
    g = lb.param_groups[0]
    assert (g["lr"], g["max_iter"], g["max_eval"], g["history_size"], g["line_search_fn"]) == (0.5, 10, 15, 5, "strong_wolfe")
    for bad in (dict(lr=0.0), dict(lr=1.0, tolerance_grad=-1.0), dict(lr=1.0, history_size=0)):
        with pytest.raises(ValueError):
            O.LBFGS.with_params(p(), **bad)
    # RAdam: threshold 5 is the fused rule; another value changes when rectification starts
    torch.manual_seed(0)
    w5, w4, wt = (torch.nn.Parameter(torch.tensor([1.0, -2.0, 3.0])) for _ in range(3))
    o5, o4, ot = O.RAdam.with_threshold([w5], 0.01, 5.0), O.RAdam.with_threshold([w4], 0.01, 4.0), torch.optim.RAdam([wt], 0.01)
    first_diff = None
    for step in range(1, 9):
        gr = torch.randn(3)
        for w, o in ((w5, o5), (w4, o4), (wt, ot)):
            w.grad = gr.clone()
            o.step()
        assert torch.allclose(w5, wt, atol=1e-6)                      # threshold 5 == torch
        if first_diff is None and not torch.allclose(w4, w5, atol=1e-7):
            first_diff = step
    # with beta2 = 0.999, rho_t passes 4 at step 5 and 5 at step 6: the two runs part at step 5
    assert first_diff == 5 and O.RAdam.with_weight_decay(p(), 1e-3, 0.1).weight_decay == pytest.approx(0.1)


def test_rust_call_forms_without_parameters():
    """``SGD::new(0.01)`` then ``optimizer.step(&param, &grad)`` (README of the reference; src/optim/mod.rs:45-60,93-137)."""
    import rustorch as rt
    import rustorch_b200.optim as O
    o = O.SGD.new(0.1)
    p, g = rt.tensor([1.0, 2.0]), rt.tensor([1.0, 1.0])
    o.step(p, g)                                                     # wrapper tensors, updated in place
    assert p.as_slice() == pytest.approx([0.9, 1.9]) and o.learning_rate == pytest.approx(0.1)
    m = O.SGD.with_momentum(0.1, 0.9)
    t = torch.ones(3)
    m.step(t, torch.ones(3))
    m.step(t, torch.ones(3))
    assert t.tolist() == pytest.approx([0.71] * 3)                    # 1 - 0.1 - 0.1 * 1.9
    a = O.Adam.default_params(0.01)
    a.step(t, torch.ones(3))
    assert t.tolist() == pytest.approx([0.70] * 3, abs=1e-6) and a.beta1 == pytest.approx(0.9)
    assert O.AdamW.default_params(1e-3).weight_decay == pytest.approx(0.01) and O.RMSprop.default_params(0.01).eps == pytest.approx(1e-8)
    assert O.NAdam.with_weight_decay(2e-3, 0.1).weight_decay == pytest.approx(0.1) and O.LBFGS.new(1.0).learning_rate == 1.0
    lin = torch.nn.Linear(2, 1)
    assert O.SGD.with_momentum(lin.parameters(), 0.1, 0.9).momentum == pytest.approx(0.9)      # parameters first still works
    sched = O.WarmupScheduler(O.SGD.new(0.01), 0.1, 5)
    for _ in range(5):
        sched.step()
    assert sched.optimizer.learning_rate == pytest.approx(0.1)
