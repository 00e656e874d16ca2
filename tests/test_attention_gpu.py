"""tcgen05 flash attention forward/backward vs fp32 math attention."""
import math

import pytest
import torch

from conftest import assert_close, rel_err

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
    assert_close(o, ref, atol_frac=8e-3, rtol=3e-2)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,T,H,Hkv,D", [(2, 256, 4, 4, 64), (1, 384, 8, 2, 128), (1, 200, 2, 2, 64), (1, 328, 4, 2, 128),
                                         (2, 72, 4, 4, 128), (1, 1160, 3, 3, 64)])
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
    assert_close(qa.grad, qr.grad, atol_frac=8e-3, rtol=3e-2)
    assert rel_err(ka.grad, kr.grad) < 3e-2
    assert_close(ka.grad, kr.grad, atol_frac=8e-3, rtol=3e-2)
    assert rel_err(va.grad, vr.grad) < 3e-2
    assert_close(va.grad, vr.grad, atol_frac=8e-3, rtol=3e-2)


def test_attention_strided_qkv_views():
    from rustorch_b200.ops import kernels as K_
    B, T, H, D = 2, 256, 4, 64
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(B, T, 3, H, D, device="cuda", generator=g).to(torch.bfloat16)
    o, _ = K_.attention_fwd(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], True)
    ref = _ref_attn(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], True)
    assert rel_err(o, ref) < 2e-2
    assert_close(o, ref, atol_frac=8e-3, rtol=3e-2)


def test_multihead_attention_masks_weights_dropout_on_native_kernels():
    """Masks, key-padding masks, need_weights and dropout take the batched tcgen05 GEMM + native softmax / dropout
    kernels (not SDPA / eager): values and gradients against the fp32 PyTorch expression of the same module."""
    from rustorch_b200 import _native
    from rustorch_b200 import nn as rnn
    torch.manual_seed(0)
    B, T, E, H = 3, 64, 128, 4
    mha = rnn.MultiheadAttention(E, H).cuda().bfloat16()
    ref = rnn.MultiheadAttention(E, H).cuda().float()
    ref.load_state_dict({k: v.float() for k, v in mha.state_dict().items()})
    x = torch.randn(B, T, E, device="cuda").bfloat16()
    attn_mask = (torch.rand(T, T, device="cuda") > 0.3).float()
    attn_mask.fill_diagonal_(1.0)
    kpm = torch.ones(B, T, device="cuda")
    kpm[:, 50:] = 0
    x1, x2 = x.clone().requires_grad_(True), x.float().requires_grad_(True)
    n0 = _native.launch_count()
    o1, w1 = mha(x1, x1, x1, key_padding_mask=kpm, need_weights=True, attn_mask=attn_mask)
    assert _native.launch_count() - n0 >= 5, "native kernels not used"
    o2, w2 = ref(x2, x2, x2, key_padding_mask=kpm, need_weights=True, attn_mask=attn_mask)
    assert rel_err(o1, o2) < 3e-2 and rel_err(w1, w2) < 3e-2
    assert float(w1[:, :, 50:].abs().max()) < 1e-6                         # padded keys get no weight
    g = torch.randn_like(o2)
    (o1.float() * g).sum().backward()
    (o2 * g).sum().backward()
    assert rel_err(x1.grad, x2.grad) < 5e-2
    assert_close(x1.grad, x2.grad, atol_frac=8e-3, rtol=3e-2)
    for (k1, p1), (_, p2) in zip(sorted(mha.named_parameters()), sorted(ref.named_parameters())):
        assert rel_err(p1.grad, p2.grad) < 5e-2, k1
    # dropout on the probabilities: native Philox kernel, expectation preserved, eval mode deterministic
    drop = rnn.MultiheadAttention(E, H, dropout=0.5).cuda().bfloat16()
    drop.train()
    n0 = _native.launch_count()
    a, _ = drop(x, need_weights=False)
    b, _ = drop(x, need_weights=False)
    assert _native.launch_count() > n0 and not torch.equal(a, b)
    drop.eval()
    c, _ = drop(x, need_weights=False)
    d, _ = drop(x, need_weights=False)
    assert torch.equal(c, d)
