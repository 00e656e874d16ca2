"""tcgen05 flash attention forward/backward vs fp32 math attention."""
import math

import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _ref_attn(q, k, v, causal):
    # q [B,T,H,D], k/v [B,Tk,Hkv,D] -> fp32 math reference
    B, T, H, D = q.shape
    Hkv = k.shape[2]
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(H // Hkv, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(H // Hkv, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    if causal:
        Tk = k.shape[1]
        mask = torch.ones(T, Tk, dtype=torch.bool, device=q.device).tril(Tk - T)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    return (p @ vf).transpose(1, 2)


def _inputs(B, T, H, Hkv, D, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h: torch.randn(B, T, h, D, device="cuda", generator=g).to(torch.bfloat16)
    return mk(H), mk(Hkv), mk(Hkv)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,T,H,Hkv,D", [(2, 256, 4, 4, 64), (1, 384, 8, 2, 128), (2, 200, 2, 2, 64),
                                         (1, 1024, 2, 1, 64)])
def test_attention_forward(causal, B, T, H, Hkv, D):
    from rustorch_b200.ops import kernels as K_
    q, k, v = _inputs(B, T, H, Hkv, D)
    o, lse = K_.attention_fwd(q, k, v, causal)
    ref = _ref_attn(q, k, v, causal)
    assert rel_err(o, ref) < 2e-2


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,T,H,Hkv,D", [(2, 256, 4, 4, 64), (1, 384, 8, 2, 128), (1, 200, 2, 2, 64)])
def test_attention_backward(causal, B, T, H, Hkv, D):
    from rustorch_b200.nn.fused import FlashAttentionFn
    q, k, v = _inputs(B, T, H, Hkv, D, seed=1)
    g = torch.Generator(device="cuda").manual_seed(5)
    do = torch.randn(B, T, H, D, device="cuda", generator=g).to(torch.bfloat16)
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    o = FlashAttentionFn.apply(qa, ka, va, causal, None)
    o.backward(do)
    qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
    _ref_attn(qr, kr, vr, causal).backward(do.float())
    assert rel_err(qa.grad, qr.grad) < 3e-2
    assert rel_err(ka.grad, kr.grad) < 3e-2
    assert rel_err(va.grad, vr.grad) < 3e-2


def test_attention_strided_qkv_views():
    from rustorch_b200.ops import kernels as K_
    B, T, H, D = 2, 256, 4, 64
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(B, T, 3, H, D, device="cuda", generator=g).to(torch.bfloat16)
    o, _ = K_.attention_fwd(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], True)
    ref = _ref_attn(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], True)
    assert rel_err(o, ref) < 2e-2
