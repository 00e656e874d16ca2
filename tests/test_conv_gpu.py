"""Implicit-GEMM conv2d (forward, weight gradient, stride-1 input gradient) vs fp32 cuDNN / ATen references."""
import pytest
import torch
import torch.nn.functional as F

from conftest import assert_close, rel_err
from rustorch_b200 import _native

pytestmark = pytest.mark.gpu

# (N, Cin, H, W, Cout, k, stride, pad): the ResNet-18/34 body shapes (scaled batch) + edge cases
CASES = [
    (4, 64, 56, 56, 64, 3, 1, 1),
    (4, 64, 56, 56, 128, 3, 2, 1),
    (4, 64, 56, 56, 128, 1, 2, 0),
    (3, 128, 28, 28, 128, 3, 1, 1),
    (5, 256, 14, 14, 256, 3, 1, 1),
    (6, 512, 7, 7, 512, 3, 1, 1),
    (2, 256, 14, 14, 512, 3, 2, 1),
    (2, 64, 19, 23, 192, 3, 1, 1),      # odd spatial sizes, Cout not a multiple of 128
    (1, 128, 9, 9, 64, 5, 1, 2),
    (2, 64, 12, 12, 64, 1, 1, 0),
    (2, 64, 112, 112, 64, 3, 1, 1),     # resident-halo kernel, two halo stages
    (3, 64, 7, 9, 128, 3, 1, 1),        # resident-halo kernel, 128 output channels per CTA, images smaller than a tile
]


@pytest.mark.parametrize("N,Cin,H,W,Cout,k,s,p", CASES)
def test_conv2d_forward_backward(N, Cin, H, W, Cout, k, s, p):
    from rustorch_b200 import _native
    from rustorch_b200.ops.conv import conv2d, supported
    torch.manual_seed(0)
    x0 = torch.randn(N, Cin, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    w0 = (torch.randn(Cout, Cin, k, k, device="cuda") * (2.0 / (Cin * k * k)) ** 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    b0 = torch.randn(Cout, device="cuda").bfloat16()
    assert supported(x0, w0, s, p)
    x, w, b = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    before = _native.launch_count()
    y = conv2d(x, w, b, s, p)
    xr, wr, br = x0.float().requires_grad_(True), w0.float().requires_grad_(True), b0.float().requires_grad_(True)
    yr = F.conv2d(xr, wr, br, s, p)
    assert y.shape == yr.shape and rel_err(y, yr) < 1e-2
    g = torch.randn_like(yr)
    y.backward(g.bfloat16())
    yr.backward(g.bfloat16().float())
    assert _native.launch_count() - before >= (3 if s == 1 else 2)
    assert rel_err(w.grad, wr.grad) < 2e-2, "wgrad"
    assert rel_err(x.grad, xr.grad) < 2e-2, "dgrad"
    assert rel_err(b.grad, br.grad) < 2e-2
    assert_close(b.grad, br.grad, atol_frac=8e-3, rtol=3e-2)
    _native.check_status()


def test_conv_module_and_resnet_block_use_native_kernels():
    from rustorch_b200 import _native, nn as rnn
    conv = rnn.Conv2d(64, 128, 3, stride=1, padding=1, bias=False).cuda().bfloat16().to(memory_format=torch.channels_last)
    x = torch.randn(2, 64, 16, 16, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    before = _native.launch_count()
    y = conv(x)
    y.float().sum().backward()
    assert _native.launch_count() - before >= 3 and x.grad is not None and conv.weight.grad is not None
    ref = F.conv2d(x.detach().float(), conv.weight.detach().float(), None, 1, 1)
    assert rel_err(y, ref) < 1e-2
    assert_close(y, ref, atol_frac=8e-3, rtol=3e-2)
    stem = rnn.Conv2d(3, 64, 7, stride=2, padding=3).cuda().bfloat16()          # 3 input channels: patch matrix + GEMM
    assert stem(torch.randn(2, 3, 32, 32, device="cuda").bfloat16()).shape == (2, 64, 16, 16)


@pytest.mark.parametrize("N,Cin,H,W,Cout,k,s,p", [(4, 3, 64, 64, 64, 7, 2, 3), (2, 3, 33, 41, 32, 3, 1, 1), (3, 12, 20, 20, 64, 4, 1, 0)])
def test_small_cin_conv_im2col_gemm(N, Cin, H, W, Cout, k, s, p):
    """Stem convolutions: patch matrix + tcgen05 GEMM forward, weight and bias gradients against fp32."""
    from rustorch_b200 import _native
    from rustorch_b200.ops.conv import conv2d, im2col_supported
    torch.manual_seed(1)
    x = torch.randn(N, Cin, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    w0 = (torch.randn(Cout, Cin, k, k, device="cuda") * (2.0 / (Cin * k * k)) ** 0.5).bfloat16()
    b0 = torch.randn(Cout, device="cuda").bfloat16()
    assert im2col_supported(x, w0, s, p)
    w, b = w0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    before = _native.launch_count()
    y = conv2d(x, w, b, s, p)
    wr, br = w0.float().requires_grad_(True), b0.float().requires_grad_(True)
    yr = F.conv2d(x.float(), wr, br, s, p)
    assert y.shape == yr.shape and rel_err(y, yr) < 1e-2
    g = torch.randn_like(yr)
    y.backward(g.bfloat16())
    yr.backward(g.bfloat16().float())
    assert _native.launch_count() - before >= 3          # im2col, forward GEMM, weight-gradient GEMM
    assert rel_err(w.grad, wr.grad) < 2e-2 and rel_err(b.grad, br.grad) < 2e-2
    assert not im2col_supported(x.clone().requires_grad_(True), w0, s, p)       # an input gradient is not provided
    _native.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("L,K,s,p", [(100, 3, 1, 1), (257, 5, 2, 2), (64, 1, 1, 0), (90, 7, 1, 3)])
def test_conv1d_native(L, K, s, p):
    from rustorch_b200.ops.conv import conv1d
    torch.manual_seed(0)
    x = torch.randn(3, 64, L, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(128, 64, K, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(128, device="cuda").bfloat16().requires_grad_(True)
    y = conv1d(x, w, b, s, p)
    dy = torch.randn_like(y)
    gx, gw, gb = torch.autograd.grad(y, (x, w, b), dy)
    xr, wr, br = (t.detach().float().cpu().requires_grad_(True) for t in (x, w, b))
    yr = F.conv1d(xr, wr, br, s, p)
    rx, rw, rb = torch.autograd.grad(yr, (xr, wr, br), dy.float().cpu())
    for got, ref in ((y, yr), (gx, rx), (gw, rw), (gb, rb)):
        assert got.shape == ref.shape
        assert rel_err(got.float().cpu(), ref) < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("K,s,p,op", [(3, 1, 1, 0), (4, 2, 1, 0), (3, 2, 1, 1), (6, 3, 2, 1), (2, 2, 0, 0)])
def test_conv_transpose2d_native(K, s, p, op):
    from rustorch_b200.ops.conv import conv_transpose2d, conv_transpose2d_supported
    torch.manual_seed(0)
    x = torch.randn(2, 64, 9, 11, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(64, 128, K, K, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(128, device="cuda").bfloat16()
    assert conv_transpose2d_supported(x, w, s, p, op, 1, 1)
    y = conv_transpose2d(x, w, b, s, p, op)
    dy = torch.randn_like(y)
    gx, gw = torch.autograd.grad(y, (x, w), dy)
    xr, wr = (t.detach().float().cpu().requires_grad_(True) for t in (x, w))
    yr = F.conv_transpose2d(xr, wr, b.float().cpu(), s, p, op)
    rx, rw = torch.autograd.grad(yr, (xr, wr), dy.float().cpu())
    for got, ref in ((y, yr), (gx, rx), (gw, rw)):
        assert got.shape == ref.shape
        assert rel_err(got.float().cpu(), ref) < 2e-2


# ---------------------------------------------------------------- generic N-d path: unfold + tcgen05 GEMM + fold
def _conv_nd_case(nd, cin, cout, k, stride, pad, dil, groups, size, seed=0):
    from rustorch_b200.ops import conv_nd as CN
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((2, cin) + (size,) * nd, device="cuda", generator=g).bfloat16()
    w = (torch.randn((cout, cin // groups) + (k,) * nd, device="cuda", generator=g) * 0.2).bfloat16()
    b = torch.randn(cout, device="cuda", generator=g).bfloat16()
    xs = [x.clone().requires_grad_(True), x.float().requires_grad_(True)]
    ws = [w.clone().requires_grad_(True), w.float().requires_grad_(True)]
    bs = [b.clone().requires_grad_(True), b.float().requires_grad_(True)]
    n0 = _native.launch_count()
    y = CN.conv_nd(xs[0], ws[0], bs[0], stride, pad, dil, groups)
    assert _native.launch_count() > n0, "native path not taken"
    ref = (F.conv1d, F.conv2d, F.conv3d)[nd - 1](xs[1], ws[1], bs[1], stride, pad, dil, groups)
    assert y.shape == ref.shape
    assert rel_err(y, ref) < 2e-2
    assert_close(y, ref, atol_frac=8e-3, rtol=3e-2)
    dy = torch.randn(ref.shape, device="cuda", generator=g)
    y.backward(dy.bfloat16())
    ref.backward(dy.bfloat16().float())
    assert rel_err(xs[0].grad, xs[1].grad) < 3e-2
    assert_close(xs[0].grad, xs[1].grad, atol_frac=8e-3, rtol=3e-2)
    assert rel_err(ws[0].grad, ws[1].grad) < 3e-2
    assert_close(ws[0].grad, ws[1].grad, atol_frac=8e-3, rtol=3e-2)
    assert rel_err(bs[0].grad, bs[1].grad) < 3e-2
    assert_close(bs[0].grad, bs[1].grad, atol_frac=8e-3, rtol=3e-2)


@pytest.mark.parametrize("nd,cin,cout,k,stride,pad,dil,groups,size", [
    (3, 16, 32, 3, 1, 1, 1, 1, 9),          # Conv3d
    (3, 16, 24, 3, 2, 1, 2, 4, 11),         # Conv3d with stride, dilation and groups (the reference kernel's feature set)
    (2, 24, 48, 3, 1, 2, 2, 3, 14),         # dilated grouped Conv2d
    (2, 12, 12, 3, 1, 1, 1, 12, 10),        # depthwise Conv2d (one channel per group)
    (1, 8, 20, 5, 2, 3, 1, 2, 33),          # grouped Conv1d, channel counts that are not multiples of 8
    (2, 3, 10, 2, 1, 0, 1, 1, 7),           # tiny channel counts, even kernel
])
def test_conv_nd_unfold_gemm_path(nd, cin, cout, k, stride, pad, dil, groups, size):
    _conv_nd_case(nd, cin, cout, k, stride, pad, dil, groups, size)


@pytest.mark.parametrize("nd,cin,cout,k,stride,pad,opad,dil,groups,size", [
    (1, 16, 24, 4, 2, 1, 0, 1, 1, 17),      # ConvTranspose1d
    (3, 8, 16, 3, 2, 1, 1, 1, 2, 5),        # ConvTranspose3d with groups and output padding
    (2, 12, 8, 3, 1, 0, 0, 2, 4, 9),        # dilated grouped ConvTranspose2d
])
def test_conv_transpose_nd_path(nd, cin, cout, k, stride, pad, opad, dil, groups, size):
    from rustorch_b200.ops import conv_nd as CN
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((2, cin) + (size,) * nd, device="cuda", generator=g).bfloat16()
    w = (torch.randn((cin, cout // groups) + (k,) * nd, device="cuda", generator=g) * 0.2).bfloat16()
    b = torch.randn(cout, device="cuda", generator=g).bfloat16()
    xs = [x.clone().requires_grad_(True), x.float().requires_grad_(True)]
    ws = [w.clone().requires_grad_(True), w.float().requires_grad_(True)]
    bs = [b.clone().requires_grad_(True), b.float().requires_grad_(True)]
    n0 = _native.launch_count()
    y = CN.conv_transpose_nd(xs[0], ws[0], bs[0], stride, pad, opad, groups, dil)
    assert _native.launch_count() > n0
    ref = (F.conv_transpose1d, F.conv_transpose2d, F.conv_transpose3d)[nd - 1](xs[1], ws[1], bs[1], stride, pad, opad, groups, dil)
    assert y.shape == ref.shape and rel_err(y, ref) < 2e-2
    dy = torch.randn(ref.shape, device="cuda", generator=g)
    y.backward(dy.bfloat16())
    ref.backward(dy.bfloat16().float())
    assert rel_err(xs[0].grad, xs[1].grad) < 3e-2 and rel_err(ws[0].grad, ws[1].grad) < 3e-2 and rel_err(bs[0].grad, bs[1].grad) < 3e-2


def test_conv3d_and_transpose_layers_use_the_native_path():
    from rustorch_b200 import nn as rnn
    torch.manual_seed(0)
    layer = rnn.Conv3d(8, 16, (3, 3, 3), stride=1, padding=1, dilation=1, groups=2).cuda().bfloat16()
    x = torch.randn(2, 8, 6, 6, 6, device="cuda").bfloat16()
    n0 = _native.launch_count()
    y = layer(x)
    assert _native.launch_count() > n0
    ref = F.conv3d(x.float(), layer.weight.float(), layer.bias.float(), 1, 1, 1, 2)
    assert rel_err(y, ref) < 2e-2
    assert_close(y, ref, atol_frac=8e-3, rtol=3e-2)
    up = rnn.ConvTranspose1d(8, 8, 4, stride=2, padding=1).cuda().bfloat16()
    z = torch.randn(2, 8, 10, device="cuda").bfloat16()
    n0 = _native.launch_count()
    out = up(z)
    assert _native.launch_count() > n0 and out.shape == (2, 8, 20)
    assert rel_err(out, F.conv_transpose1d(z.float(), up.weight.float(), up.bias.float(), 2, 1)) < 2e-2
