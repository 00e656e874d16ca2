"""Native elementwise / activation / softmax / row-reduction kernels vs fp32 PyTorch references."""
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_err

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16, torch.float16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 8e-3, torch.float16: 2e-3}


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("n", [1, 7, 4096, 1000003])
def test_binary_ops(dtype, n):
    from rustorch_b200.ops import elementwise as ew
    torch.manual_seed(0)
    a = torch.randn(n, device="cuda").to(dtype)
    b = (torch.rand(n, device="cuda") + 0.5).to(dtype)
    for name, ref in (("add", lambda x, y: x + 0.5 * y), ("sub", lambda x, y: x - 0.5 * y), ("mul", lambda x, y: x * y),
                      ("div", lambda x, y: x / y), ("max", torch.maximum), ("min", torch.minimum)):
        alpha = 0.5 if name in ("add", "sub") else 1.0
        out = ew.binary(name, a, b, alpha)
        assert out.dtype == dtype and rel_err(out, ref(a.float(), b.float())) < TOL[dtype], name
        outs = ew.binary(name, a, 1.5, alpha)
        assert rel_err(outs, ref(a.float(), torch.full_like(a, 1.5).float())) < TOL[dtype], name
    assert rel_err(ew.binary("pow", b, 2.0), b.float() ** 2) < TOL[dtype]


@pytest.mark.parametrize("dtype", DT)
def test_unary_forward_backward(dtype):
    from rustorch_b200.ops import elementwise as ew
    torch.manual_seed(1)
    x0 = (torch.randn(3, 1001, device="cuda") * 2).to(dtype)
    pos_only = {"log", "sqrt", "rsqrt", "reciprocal"}
    for name in ("relu", "sigmoid", "tanh", "gelu_tanh", "gelu_erf", "silu", "elu", "leaky_relu", "selu", "mish", "softplus",
                 "hardtanh", "relu6", "hardsigmoid", "hardswish", "exp", "log", "sqrt", "rsqrt", "neg", "abs", "square",
                 "sin", "cos", "reciprocal"):
        xb = (x0.float().abs() + 0.5).to(dtype) if name in pos_only else x0
        x = xb.clone().requires_grad_(True)
        y = ew.unary(name, x)
        xr = xb.float().clone().requires_grad_(True)
        d0, d1 = ew._DEFAULTS.get(name, (0.0, 0.0))
        yr = ew._torch_unary(name, xr, d0, d1)
        assert y.dtype == dtype and rel_err(y, yr) < TOL[dtype], name
        g = torch.randn_like(yr)
        y.backward(g.to(dtype))
        yr.backward(g.to(dtype).float())
        assert rel_err(x.grad, xr.grad) < 2 * TOL[dtype], name


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("C", [5, 128, 300, 1024, 5000, 50257])
def test_softmax_and_log_softmax(dtype, C):
    from rustorch_b200.ops import elementwise as ew
    torch.manual_seed(2)
    x0 = (torch.randn(37, C, device="cuda") * 3).to(dtype)
    for fn, ref in ((ew.softmax, F.softmax), (ew.log_softmax, F.log_softmax)):
        x = x0.clone().requires_grad_(True)
        xr = x0.float().clone().requires_grad_(True)
        y, yr = fn(x, -1), ref(xr, -1)
        assert rel_err(y, yr) < TOL[dtype]
        g = torch.randn_like(yr)
        y.backward(g.to(dtype))
        yr.backward(g.to(dtype).float())
        assert rel_err(x.grad, xr.grad) < 3 * TOL[dtype]
    # other dims and masked rows
    x3 = torch.randn(4, 6, 9, device="cuda").to(dtype)
    assert rel_err(ew.softmax(x3, 1), F.softmax(x3.float(), 1)) < TOL[dtype]
    xm = torch.full((2, 40), float("-inf"), device="cuda", dtype=dtype)
    xm[1, 3] = 1.0
    sm = ew.softmax(xm)
    assert torch.isfinite(sm).all() and sm[0].sum() == 0 and sm[1, 3] == 1


@pytest.mark.parametrize("dtype", DT)
def test_row_reductions(dtype):
    from rustorch_b200.ops import elementwise as ew
    x = torch.randn(33, 777, device="cuda").to(dtype)
    xf = x.float()
    assert rel_err(ew.reduce_last(x, "sum"), xf.sum(-1)) < 1e-4
    assert rel_err(ew.reduce_last(x, "mean"), xf.mean(-1)) < 1e-4
    assert torch.equal(ew.reduce_last(x, "max"), xf.max(-1).values) and torch.equal(ew.reduce_last(x, "min"), xf.min(-1).values)
    assert rel_err(ew.reduce_last(x, "var"), xf.var(-1)) < 1e-4
    assert rel_err(ew.reduce_last(x, "var", unbiased=False), xf.var(-1, unbiased=False)) < 1e-4


def test_nn_activations_use_native_kernels():
    from rustorch_b200 import _native, nn as rnn
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    before = _native.launch_count()
    y = rnn.GELU()(x)
    rnn.Softmax(-1)(y).sum().backward()
    assert _native.launch_count() - before >= 4          # gelu fwd/bwd + softmax fwd/bwd
    assert x.grad is not None


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("shape", [(32, 64), (8, 64, 14, 14), (4, 16, 9, 7), (2, 8, 5, 6, 7), (6, 128, 33)])
@pytest.mark.parametrize("fuse", [False, True])
def test_batchnorm_training_forward_backward(dtype, shape, fuse):
    from rustorch_b200.ops.batchnorm import batch_norm
    torch.manual_seed(3)
    C = shape[1]
    x0 = (torch.randn(*shape, device="cuda") * 2 + 0.5).to(dtype)
    res0 = torch.randn(*shape, device="cuda").to(dtype) if fuse else None
    w0, b0 = torch.rand(C, device="cuda") + 0.5, torch.randn(C, device="cuda")
    rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    rm_r, rv_r = rm.clone(), rv.clone()
    x, w, b = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    res = res0.clone().requires_grad_(True) if fuse else None
    y = batch_norm(x, rm, rv, w, b, True, 0.1, 1e-5, res, fuse)
    xr, wr, br = x0.float().clone().requires_grad_(True), w0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    resr = res0.float().clone().requires_grad_(True) if fuse else None
    yr = F.batch_norm(xr, rm_r, rv_r, wr, br, True, 0.1, 1e-5)
    if fuse:
        yr = torch.relu(yr + resr)
    tol = TOL[dtype] * 2
    assert y.shape == yr.shape and rel_err(y, yr) < tol
    assert rel_err(rm, rm_r) < 1e-3 and rel_err(rv, rv_r) < 1e-3
    g = torch.randn_like(yr)
    y.backward(g.to(dtype))
    yr.backward(g.to(dtype).float())
    assert rel_err(x.grad, xr.grad) < 4 * tol
    assert rel_err(w.grad, wr.grad) < 4 * tol and rel_err(b.grad, br.grad) < 4 * tol
    if fuse:
        assert rel_err(res.grad, resr.grad) < tol


def test_batchnorm_eval_and_module():
    from rustorch_b200 import nn as rnn
    bn = rnn.BatchNorm2d(32).cuda()
    ref = torch.nn.BatchNorm2d(32).cuda()
    x = torch.randn(4, 32, 10, 10, device="cuda")
    for _ in range(3):
        y, yr = bn(x), ref(x)
    assert rel_err(y, yr) < 1e-4 and rel_err(bn.running_var, ref.running_var) < 1e-4 and int(bn.num_batches_tracked) == 3
    bn.eval(), ref.eval()
    xe = x.clone().requires_grad_(True)
    xer = x.clone().requires_grad_(True)
    ye, yer = bn(xe), ref(xer)
    assert rel_err(ye, yer) < 1e-4
    ye.sum().backward(), yer.sum().backward()
    assert rel_err(xe.grad, xer.grad) < 1e-4
    xcl = x.to(memory_format=torch.channels_last)
    assert rel_err(bn(xcl), yer) < 1e-4
