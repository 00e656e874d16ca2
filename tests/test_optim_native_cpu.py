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


def test_flat_params_keep_channels_last_filters_in_physical_order():
    from rustorch_b200.optim.flat import FlatParams
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Conv2d(4, 8, 3), torch.nn.Conv2d(8, 8, 1), torch.nn.Linear(8, 2)).to(memory_format=torch.channels_last)
    w0 = m[0].weight.detach().clone()
    flat = FlatParams(m)
    assert m[0].weight._flat_ohwi and not m[2].weight._flat_ohwi
    assert torch.equal(m[0].weight.data, w0) and m[0].weight.data.is_contiguous(memory_format=torch.channels_last)
    # the flat slice IS the [Cout, KH, KW, Cin] array
    _, p, o, k = next(e for e in flat.entries if e[0] == "0.weight")
    assert torch.equal(flat.lp[o:o + k].view(8, 3, 3, 4), w0.permute(0, 2, 3, 1))
    x = torch.randn(2, 4, 6, 6).contiguous(memory_format=torch.channels_last)
    m[2](m[1](m[0](x)).mean((2, 3))).sum().backward()
    g0 = m[0].weight.grad.clone()
    assert flat.collect_autograd_grads() == 6
    assert torch.allclose(flat.named_views(flat.grad)["0.weight"], g0)
    assert torch.allclose(m[0].weight.main_grad.view(8, 3, 3, 4), g0.permute(0, 2, 3, 1))


def test_split_k_rule_fills_one_wave():
    """Weight-gradient GEMMs split the contraction so that tiles x splits stay within one wave of 148 CTAs."""
    from rustorch_b200.nn import fused
    from rustorch_b200.distributed.tp_fused import _wgrad_splits
    sms = fused._num_sms()
    for tiles, kb in ((72, 256), (54, 256), (18, 256), (1, 4096), (147, 256), (148, 256), (1179, 256), (6, 16)):
        sk = fused._split_k_for(tiles, kb)
        assert sk >= 1 and (tiles >= sms or tiles * sk <= sms) and sk <= max(1, kb // 8)
        if tiles < sms and kb >= 8 * (sms // tiles):
            assert tiles * (sk + 1) > sms                # as many splits as fit
    assert fused._split_k_for(72, 256) == sms // 72
    assert _wgrad_splits(3072, 768, 16384) == fused._split_k_for(24 * 3, 256)
    assert _wgrad_splits(50304, 768, 16384) == 1
