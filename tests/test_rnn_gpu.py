"""Whole-sequence recurrent layers on the GPU: bf16 through the tcgen05 GEMM + fused gate kernels against the fp32
torch.nn module with the same weights; fp32 through the gate kernels against torch.nn exactly."""
import pytest
import torch

from conftest import rel_err
from rustorch_b200 import _native
from rustorch_b200 import nn as rnn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["LSTM", "GRU", "RNN"])
@pytest.mark.parametrize("kw", [dict(), dict(num_layers=2, bidirectional=True, batch_first=True)])
def test_bf16_sequence_layers_on_native_kernels(kind, kw):
    torch.manual_seed(0)
    ours = getattr(rnn, kind)(64, 128, **kw).cuda().bfloat16()
    ref = getattr(torch.nn, kind)(64, 128, **kw).cuda().float()
    ref.load_state_dict({k: v.float() for k, v in ours.state_dict().items()})
    B, T = 16, 12
    x = torch.randn((B, T, 64) if kw.get("batch_first") else (T, B, 64), device="cuda").bfloat16()
    x1, x2 = x.clone().requires_grad_(True), x.float().requires_grad_(True)
    n0 = _native.launch_count()
    o1, s1 = ours(x1)
    o2, s2 = ref(x2)
    assert rel_err(o1, o2) < 3e-2
    s1 = s1 if isinstance(s1, tuple) else (s1,)
    s2 = s2 if isinstance(s2, tuple) else (s2,)
    for a, b in zip(s1, s2):
        assert rel_err(a, b) < 3e-2
    w = torch.randn_like(o2)
    (o1.float() * w).sum().backward()
    (o2 * w).sum().backward()
    layers = kw.get("num_layers", 1) * (2 if kw.get("bidirectional") else 1)
    # per layer and direction: 1 projection GEMM + T x (GEMM + gate kernel) forward, and as many again backward
    assert _native.launch_count() - n0 >= layers * (2 * T + 1) * 2, "the native kernels did not run"
    assert rel_err(x1.grad, x2.grad) < 5e-2
    for (k, p), (_, q) in zip(sorted(ours.named_parameters()), sorted(ref.named_parameters())):
        assert rel_err(p.grad, q.grad) < 5e-2, k


@pytest.mark.parametrize("kind", ["LSTM", "GRU"])
def test_fp32_sequence_layers_gate_kernels(kind):
    torch.manual_seed(1)
    ours = getattr(rnn, kind)(24, 40, num_layers=2).cuda()
    ref = getattr(torch.nn, kind)(24, 40, num_layers=2).cuda()
    ref.load_state_dict(ours.state_dict())
    x = torch.randn(9, 5, 24, device="cuda")
    x1, x2 = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    prev, prev_dnn = torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = torch.backends.cudnn.allow_tf32 = False      # full fp32 in the oracle too
    try:
        o1, _ = ours(x1)
        o2, _ = ref(x2)
        o1.square().sum().backward()
        o2.square().sum().backward()
    finally:
        torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = prev, prev_dnn
    torch.testing.assert_close(o1, o2, rtol=5e-4, atol=5e-5)
    torch.testing.assert_close(x1.grad, x2.grad, rtol=2e-3, atol=2e-4)
    for (k, p), (_, q) in zip(sorted(ours.named_parameters()), sorted(ref.named_parameters())):
        torch.testing.assert_close(p.grad, q.grad, rtol=2e-3, atol=2e-4, msg=lambda m, k=k: f"{k}: {m}")
