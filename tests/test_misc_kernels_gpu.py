"""Pooling, dropout, recurrent gate, AMP unscale and CSR kernels against PyTorch fp32 references."""
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("k,s,p", [(3, 2, 1), (2, 2, 0), (3, 1, 1), ((2, 3), (1, 2), (1, 0))])
def test_max_and_avg_pool_forward_backward(dtype, k, s, p):
    from rustorch_b200 import _native
    from rustorch_b200.ops import pool
    x = torch.randn(3, 16, 13, 14, device="cuda").to(dtype).contiguous(memory_format=torch.channels_last)
    for ours, ref in ((pool.max_pool2d, F.max_pool2d), (pool.avg_pool2d, F.avg_pool2d)):
        # fp32 reference on the CPU, on a plain NCHW tensor
        xa, xb = x.clone().requires_grad_(True), x.float().cpu().contiguous().clone().requires_grad_(True)
        ya, yb = ours(xa, k, s, p), ref(xb, k, s, p)
        assert ya.shape == yb.shape and rel_err(ya.cpu(), yb) < (1e-6 if dtype == torch.float32 else 8e-3)
        g = torch.randn_like(yb)
        ya.backward(g.to(dtype).cuda())
        yb.backward(g)
        assert rel_err(xa.grad.cpu(), xb.grad) < (1e-6 if dtype == torch.float32 else 1e-2)
    _native.check_status()


def test_resnet_stem_pool_and_global_pool_shapes():
    from rustorch_b200.nn import layers as L
    x = torch.randn(4, 64, 112, 112, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    y = L.MaxPool2d(3, 2, 1)(x)
    assert y.shape == (4, 64, 56, 56) and rel_err(y, F.max_pool2d(x.float(), 3, 2, 1)) < 1e-6
    z = torch.randn(4, 512, 7, 7, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    g = L.AdaptiveAvgPool2d.global_pool()(z)
    assert g.shape == (4, 512, 1, 1) and rel_err(g, z.float().mean((2, 3), keepdim=True)) < 8e-3
    g.sum().backward()
    assert rel_err(z.grad, torch.full_like(z, 1 / 49.0)) < 8e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dropout_rate_scaling_and_backward_mask(dtype):
    from rustorch_b200.ops import pool
    torch.manual_seed(123)
    x = torch.ones(1 << 20, device="cuda", dtype=dtype, requires_grad=True)
    y = pool.dropout(x, 0.3, True)
    kept = (y != 0).float().mean().item()
    assert abs(kept - 0.7) < 5e-3                                  # rate
    assert torch.allclose(y[y != 0].float(), torch.tensor(1 / 0.7, device="cuda"), rtol=1e-2)
    y.backward(torch.ones_like(y))
    assert torch.equal(x.grad != 0, y != 0)                        # backward regenerates the same mask
    y2 = pool.dropout(x.detach(), 0.3, True)
    assert not torch.equal(y2 != 0, y != 0)                        # a new call draws new bits
    assert pool.dropout(x, 0.3, False) is x


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lstm_and_gru_cells_match_pytorch(dtype):
    from rustorch_b200.nn import rnn as R
    torch.manual_seed(0)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    for cell_cls, ref_cls in ((R.LSTMCell, torch.nn.LSTMCell), (R.GRUCell, torch.nn.GRUCell)):
        cell = cell_cls(48, 64).cuda().to(dtype)
        ref = ref_cls(48, 64).cuda().float()
        ref.load_state_dict({k: v.float() for k, v in cell.state_dict().items()})
        x = torch.randn(10, 48, device="cuda").to(dtype)
        h0 = torch.randn(10, 64, device="cuda").to(dtype)
        if cell_cls is R.LSTMCell:
            c0 = torch.randn(10, 64, device="cuda").to(dtype)
            h, c = cell(x, (h0, c0))
            hr, cr = ref(x.float(), (h0.float(), c0.float()))
            assert rel_err(h, hr) < tol and rel_err(c, cr) < tol
            (h.float().sum() + (c.float() * 0.5).sum()).backward()
            (hr.sum() + (cr * 0.5).sum()).backward()
        else:
            h = cell(x, h0)
            hr = ref(x.float(), h0.float())
            assert rel_err(h, hr) < tol
            h.float().pow(2).sum().backward()
            hr.pow(2).sum().backward()
        for (n, pa), (_, pb) in zip(cell.named_parameters(), ref.named_parameters()):
            assert rel_err(pa.grad, pb.grad) < (1e-4 if dtype == torch.float32 else 6e-2), n


def test_amp_unscale_flags_overflow_and_scales():
    from rustorch_b200.amp import GradScaler
    p = [torch.nn.Parameter(torch.zeros(1000, device="cuda")), torch.nn.Parameter(torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16))]
    sc = GradScaler(init_scale=1024.0)
    for q in p:
        q.grad = torch.full_like(q, 2048.0)
    assert sc.unscale_grads(p) is False
    assert all(torch.allclose(q.grad.float(), torch.full_like(q, 2.0).float()) for q in p)
    sc2 = GradScaler(init_scale=1024.0)
    p[1].grad[3, 5] = float("inf")
    assert sc2.unscale_grads(p) is True


def test_csr_spmv_spmm_match_dense():
    from rustorch_b200.sparse import SparseTensor
    torch.manual_seed(1)
    dense = torch.randn(300, 257, device="cuda") * (torch.rand(300, 257, device="cuda") < 0.05)
    sp = SparseTensor.from_dense(dense).to_csr()
    v, m = torch.randn(257, device="cuda"), torch.randn(257, 70, device="cuda")
    assert rel_err(sp.spmv(v), dense @ v) < 1e-5
    assert rel_err(sp.spmm(m), dense @ m) < 1e-5


def test_rope_split_and_swiglu_forward_backward():
    from rustorch_b200.models.llama import _RopeSplit, _SwiGLU, apply_rope, rope_tables
    B, T, H, Hkv, D = 2, 48, 4, 2, 64
    cos, sin = rope_tables(64, D, 10000.0, "cuda")
    qkv = torch.randn(B * T, (H + 2 * Hkv) * D, device="cuda").bfloat16()
    a, b = qkv.clone().requires_grad_(True), qkv.float().clone().requires_grad_(True)
    q, k, v = _RopeSplit.apply(a, cos, sin, B, T, H, Hkv, D)
    r = b.view(B, T, H + 2 * Hkv, D)
    qr, kr, vr = apply_rope(r[:, :, :H], cos, sin), apply_rope(r[:, :, H:H + Hkv], cos, sin), r[:, :, H + Hkv:]
    assert rel_err(q, qr) < 8e-3 and rel_err(k, kr) < 8e-3 and torch.equal(v.float(), vr.detach().bfloat16().float())
    gq, gk, gv = torch.randn_like(qr), torch.randn_like(kr), torch.randn_like(vr)
    torch.autograd.backward([q, k, v], [gq.bfloat16(), gk.bfloat16(), gv.bfloat16()])
    torch.autograd.backward([qr, kr, vr], [gq, gk, gv])
    assert rel_err(a.grad, b.grad) < 1e-2
    gu = torch.randn(100, 2 * 264, device="cuda").bfloat16()
    a, b = gu.clone().requires_grad_(True), gu.float().clone().requires_grad_(True)
    y = _SwiGLU.apply(a)
    yr = F.silu(b[:, :264]) * b[:, 264:]
    assert rel_err(y, yr) < 8e-3
    g = torch.randn_like(yr)
    y.backward(g.bfloat16())
    yr.backward(g)
    assert rel_err(a.grad, b.grad) < 1.5e-2


def test_llama_model_native_path_matches_fp32_reference():
    from rustorch_b200.models.llama import LlamaModel, LlamaTrainConfig
    torch.manual_seed(3)
    cfg = LlamaTrainConfig.tiny(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, n_ff=512, vocab_size=512)
    m = LlamaModel(cfg, device="cuda", dtype=torch.bfloat16)
    ref = LlamaModel(cfg, device="cuda", dtype=torch.float32)
    ref.load_state_dict({k: v.float() for k, v in m.state_dict().items()})
    idx = torch.randint(0, 512, (2, 128), device="cuda")
    tgt = idx.roll(-1, 1)
    _, la = m(idx, tgt)
    _, lb = ref(idx, tgt)
    assert abs(float(la) - float(lb)) < 3e-2
    la.backward()
    lb.backward()
    for (n, pa), (_, pb) in zip(m.named_parameters(), ref.named_parameters()):
        ga = pa.grad if pa.grad is not None else getattr(pa, "main_grad", None)
        if ga is not None and pb.grad is not None:
            assert rel_err(ga, pb.grad) < 8e-2, n


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,groups", [((4, 32, 14, 14), 8), ((3, 12, 7, 5), 4), ((2, 16, 33), 16), ((5, 6, 3, 4, 4), 3)])
def test_group_norm_native(dtype, shape, groups):
    from rustorch_b200.ops.groupnorm import group_norm
    torch.manual_seed(0)
    x = (torch.randn(*shape, device="cuda") * 2 + 0.5).to(dtype).requires_grad_(True)
    w = (torch.rand(shape[1], device="cuda") + 0.5).to(dtype).requires_grad_(True)
    b = torch.randn(shape[1], device="cuda").to(dtype).requires_grad_(True)
    dy = torch.randn(*shape, device="cuda").to(dtype)
    y = group_norm(x, groups, w, b, 1e-5)
    gx, gw, gb = torch.autograd.grad(y, (x, w, b), dy)
    xr, wr, br = (t.detach().cpu().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.group_norm(xr, groups, wr, br, 1e-5)
    rx, rw, rb = torch.autograd.grad(yr, (xr, wr, br), dy.cpu().float())
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    for got, ref in ((y, yr), (gx, rx), (gw, rw), (gb, rb)):
        err = (got.detach().cpu().float() - ref.detach()).abs().max() / ref.detach().abs().max().clamp_min(1e-6)
        assert float(err) < tol, float(err)


@pytest.mark.gpu
def test_instance_norm_layers_native():
    from rustorch_b200 import nn as rnn
    torch.manual_seed(1)
    for layer, shape in ((rnn.InstanceNorm1d(8, affine=True), (3, 8, 50)), (rnn.InstanceNorm2d(6), (2, 6, 9, 11)),
                         (rnn.InstanceNorm3d(4, affine=True), (2, 4, 3, 5, 6))):
        layer = layer.cuda()
        x = torch.randn(*shape, device="cuda", requires_grad=True)
        y = layer(x)
        y.square().sum().backward()
        xr = x.detach().cpu().requires_grad_(True)
        yr = torch.nn.functional.instance_norm(xr, None, None, None if layer.weight is None else layer.weight.detach().cpu(),
                                               None if layer.bias is None else layer.bias.detach().cpu(), True, 0.0, layer.eps)
        yr.square().sum().backward()
        assert torch.allclose(y.detach().cpu(), yr.detach(), atol=1e-4, rtol=1e-4)
        assert torch.allclose(x.grad.cpu(), xr.grad, atol=2e-3, rtol=1e-3)
