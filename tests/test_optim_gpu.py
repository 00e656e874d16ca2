"""Multi-tensor optimizer kernel (csrc/optim/multi_tensor_optim.cu) against torch.optim / fp32 torch math."""
import copy

import pytest
import torch

from rustorch_b200 import optim as O
from rustorch_b200.optim import multi_tensor

pytestmark = pytest.mark.gpu

SHAPES = [(257,), (64, 33), (4096,), (5000, 3), (1,), (12, 12, 3)] + [(17 + i,) for i in range(34)]   # 40 tensors: two launches


def _params(dtype=torch.float32, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return [torch.nn.Parameter(torch.randn(s, device="cuda", generator=g).to(dtype)) for s in SHAPES]


def _set_grads(ps, step, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(100 + step)
    for p in ps:
        p.grad = (torch.randn(p.shape, device="cuda", generator=g) * scale).to(p.dtype)


CASES = [
    ("Adam", dict(lr=1e-2, weight_decay=0.01), "Adam", {}),
    ("AdamW", dict(lr=1e-2, weight_decay=0.1), "AdamW", {}),
    ("SGD", dict(lr=0.05, momentum=0.9, weight_decay=1e-3, nesterov=True), "SGD", {}),
    ("SGD", dict(lr=0.05), "SGD", {}),
    ("NAdam", dict(lr=1e-2, weight_decay=0.01), "NAdam", {}),
    ("RAdam", dict(lr=1e-2, weight_decay=0.01), "RAdam", {}),
    ("Adamax", dict(lr=2e-2, weight_decay=0.01), "Adamax", {}),
    ("RMSprop", dict(lr=1e-2, momentum=0.9, centered=True, weight_decay=0.01), "RMSprop", {}),
    ("RMSprop", dict(lr=1e-2), "RMSprop", {}),
    ("AdaGrad", dict(lr=5e-2, lr_decay=0.01, weight_decay=0.01, initial_accumulator_value=0.1), "Adagrad", {}),
]


@pytest.mark.parametrize("name,kw,tname,tkw", CASES)
def test_multi_tensor_step_matches_torch_optim(name, kw, tname, tkw):
    ps = _params()
    ref_ps = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    ours = getattr(O, name)(ps, **kw)
    ref = getattr(torch.optim, tname)(ref_ps, **kw, **tkw)
    n0 = multi_tensor.launches
    for step in range(8):              # RAdam switches to the rectified branch at step 6
        _set_grads(ps, step)
        _set_grads(ref_ps, step)
        ours.step()
        ref.step()
    assert multi_tensor.launches - n0 == 8 * 2, "the native multi-tensor path did not run"
    for p, r in zip(ps, ref_ps):
        torch.testing.assert_close(p.data, r.data, rtol=1e-4, atol=2e-5)
    # state dict keeps torch's layout: a torch optimizer of the same kind loads it and continues identically
    sd = ours.state_dict()
    ref2_ps = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    ref2 = getattr(torch.optim, tname)(ref2_ps, **kw, **tkw)
    ref2.load_state_dict(copy.deepcopy(sd))
    _set_grads(ps, 99)
    _set_grads(ref2_ps, 99)
    ours.step()
    ref2.step()
    for p, r in zip(ps, ref2_ps):
        torch.testing.assert_close(p.data, r.data, rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("name,kw", [("LAMB", dict(lr=1e-2, weight_decay=0.01)), ("AdaBound", dict(lr=1e-2, final_lr=0.1, weight_decay=0.01))])
def test_lamb_adabound_native_match_per_tensor_math(name, kw):
    ps = _params()
    ref_ps = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    ours = getattr(O, name)(ps, **kw)
    ref = getattr(O, name)(ref_ps, **kw)
    n0 = multi_tensor.launches
    for step in range(5):
        _set_grads(ps, step)
        _set_grads(ref_ps, step)
        ours.step()
        ref._fallback_step()           # the per-tensor fp32 torch arithmetic
    assert multi_tensor.launches > n0
    for p, r in zip(ps, ref_ps):
        torch.testing.assert_close(p.data, r.data, rtol=1e-4, atol=1e-5)


def test_multi_tensor_bf16_parameters_fp32_state():
    ps = _params(torch.bfloat16)
    ref_ps = [torch.nn.Parameter(p.detach().float()) for p in ps]
    ours = O.AdamW(ps, lr=1e-2, weight_decay=0.1)
    ref = torch.optim.AdamW(ref_ps, lr=1e-2, weight_decay=0.1)
    for step in range(3):
        _set_grads(ps, step)
        for p, r in zip(ps, ref_ps):
            r.grad = p.grad.float()
        ours.step()
        ref.step()
        for p, r in zip(ps, ref_ps):    # keep the oracle on the bf16 grid the kernel rounds to
            r.data.copy_(r.data.bfloat16().float())
    assert ours.state[ps[0]]["exp_avg"].dtype == torch.float32
    for p, r in zip(ps, ref_ps):
        torch.testing.assert_close(p.data.float(), r.data, rtol=2e-2, atol=2e-2)


def test_multi_tensor_falls_back_for_cpu_and_amsgrad():
    p_cpu = [torch.nn.Parameter(torch.randn(8))]
    o = O.Adam(p_cpu, lr=1e-2)
    p_cpu[0].grad = torch.ones(8)
    n0 = multi_tensor.launches
    o.step()
    ps = _params()[:3]
    o2 = O.Adam(ps, lr=1e-2, amsgrad=True)
    _set_grads(ps, 0)
    before = ps[0].detach().clone()
    o2.step()
    assert multi_tensor.launches == n0 and not torch.equal(ps[0].data, before)
