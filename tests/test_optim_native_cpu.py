"""Native host optimizer steps (csrc/runtime/cpu_optim.cpp) against torch.optim on the same gradients."""
import pytest
import torch

from rustorch_b200 import optim as O


@pytest.mark.parametrize("name,kw", [
    ("Adam", dict(lr=1e-2, weight_decay=0.01)),
    ("AdamW", dict(lr=1e-2, weight_decay=0.1)),
    ("Adamax", dict(lr=2e-2, weight_decay=0.01)),
    ("NAdam", dict(lr=1e-2, weight_decay=0.01)),
    ("RAdam", dict(lr=1e-2, weight_decay=0.01)),
])
def test_native_step_matches_torch(name, kw):
    torch.manual_seed(0)
    p0 = torch.randn(257)
    grads = [torch.randn(257) for _ in range(12)]
    ours_p = p0.clone()
    ours = getattr(O, name)([torch.nn.Parameter(p0.clone())], **kw)
    ref_p = torch.nn.Parameter(p0.clone())
    ref = getattr(torch.optim, name)([ref_p], **kw)
    for g in grads:
        ours.step_tensor(ours_p, g)
        ref_p.grad = g.clone()
        ref.step()
    assert "_fast_state" in ours.__dict__, "native path was not taken"
    torch.testing.assert_close(ours_p, ref_p.data, rtol=2e-5, atol=2e-6)


def test_native_step_falls_back_for_double():
    p = torch.randn(16, dtype=torch.float64)
    opt = O.Adam([torch.nn.Parameter(p.clone())], lr=1e-2)
    before = p.clone()
    opt.step_tensor(p, torch.ones_like(p))
    assert "_fast_state" not in opt.__dict__ or not opt.__dict__["_fast_state"]
    assert not torch.equal(p, before)


def test_lbfgs_step_tensor_minimises_quadratic():
    torch.manual_seed(1)
    a = torch.rand(64) * 4 + 0.5                         # f(x) = 0.5 * sum(a * (x - 1)^2)
    x = torch.zeros(64)
    opt = O.LBFGS([torch.nn.Parameter(x.clone())], lr=0.2, history_size=8)
    f0 = float(0.5 * (a * (x - 1) ** 2).sum())
    for _ in range(40):
        opt.step_tensor(x, a * (x - 1))
    f1 = float(0.5 * (a * (x - 1) ** 2).sum())
    assert f1 < 1e-3 * f0
    st = next(iter(opt.__dict__["_fast_state"].values()))
    assert st["count"] == 8 and st["has_prev"] == 1


def test_lbfgs_native_matches_python_two_loop():
    torch.manual_seed(2)
    a = torch.rand(32) * 3 + 0.5
    x1, x2 = torch.zeros(32), torch.zeros(32, dtype=torch.float64)
    o1 = O.LBFGS([torch.nn.Parameter(x1.clone())], lr=0.3, history_size=4)
    o2 = O.LBFGS([torch.nn.Parameter(x2.clone())], lr=0.3, history_size=4)
    for _ in range(6):
        o1.step_tensor(x1, a * (x1 - 1))
        o2.step_tensor(x2, a.double() * (x2 - 1))
    torch.testing.assert_close(x1, x2.float(), rtol=1e-3, atol=1e-4)
