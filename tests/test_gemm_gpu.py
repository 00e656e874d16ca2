"""tcgen05 GEMM vs an fp32 PyTorch matmul of the same bf16 inputs."""
import pytest
import torch

from conftest import assert_close, rel_err

pytestmark = pytest.mark.gpu


def _mk(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * 0.5).to(torch.bfloat16)


def _ref(a, b, a_mn, b_mn):
    A = a.float().transpose(-1, -2) if a_mn else a.float()
    B = b.float() if b_mn else b.float().transpose(-1, -2)
    return A @ B


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 768, 1024),
                                   (200, 136, 72), (1000, 264, 520), (64, 8, 8)])
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    from rustorch_b200.ops import kernels as K_
    a = _mk((K, M) if a_mn else (M, K), 1)
    b = _mk((K, N) if b_mn else (N, K), 2)
    out = K_.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    ref = _ref(a, b, a_mn, b_mn)
    assert rel_err(out, ref) < 1.5e-2
    assert_close(out, ref, atol_frac=4e-3, rtol=3e-2)


@pytest.mark.parametrize("block_n", [128, 256])
def test_gemm_block_n_and_fp32_out(block_n):
    from rustorch_b200.ops import kernels as K_
    a, b = _mk((512, 320), 3), _mk((640, 320), 4)
    out = K_.gemm(a, b, out_dtype=torch.float32, block_n=block_n)
    assert rel_err(out, _ref(a, b, False, False)) < 2e-3


def test_gemm_batched_strided():
    from rustorch_b200.ops import kernels as K_
    big = _mk((4, 256, 3 * 128), 5)
    a = big[:, :, 0:128]                 # strided view, row stride 384
    b = _mk((4, 192, 128), 6)
    out = K_.gemm(a, b)
    assert rel_err(out, a.float() @ b.float().transpose(1, 2)) < 1.5e-2


def test_gemm_bias_gelu_residual_epilogues():
    from rustorch_b200.ops import kernels as K_
    M, N, K = 512, 768, 256
    a, b = _mk((M, K), 7), _mk((N, K), 8)
    bias = _mk((N,), 9)
    res = _mk((M, N), 10)
    lin = a.float() @ b.float().t() + bias.float()
    out = K_.gemm(a, b, bias=bias)
    assert rel_err(out, lin) < 1.5e-2
    assert_close(out, lin, atol_frac=4e-3, rtol=3e-2)
    out = K_.gemm(a, b, bias=bias, aux=res, epilogue=K_.EPI_RESIDUAL)
    assert rel_err(out, lin + res.float()) < 1.5e-2
    pre = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    act = K_.gemm(a, b, bias=bias, aux=pre, epilogue=K_.EPI_GELU_DUAL)
    assert rel_err(pre, lin) < 1.5e-2
    assert_close(pre, lin, atol_frac=4e-3, rtol=3e-2)
    assert rel_err(act, torch.nn.functional.gelu(lin, approximate="tanh")) < 2e-2
    # dGELU epilogue: out = (a @ b^T) * gelu'(pre)
    x = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(x, approximate="tanh").sum().backward()
    out = K_.gemm(a, b, aux=pre, epilogue=K_.EPI_DGELU)
    assert rel_err(out, (a.float() @ b.float().t()) * x.grad) < 2e-2


@pytest.mark.parametrize("split_k", [1, 4, 7])
def test_gemm_wgrad_split_k_accumulate(split_k):
    from rustorch_b200.ops import kernels as K_
    tokens, n_out, n_in = 2048, 384, 256
    dy, x = _mk((tokens, n_out), 11), _mk((tokens, n_in), 12)
    acc = torch.ones(n_out, n_in, dtype=torch.float32, device="cuda")
    K_.gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True, split_k=split_k)
    ref = 1.0 + dy.float().t() @ x.float()
    assert rel_err(acc, ref) < 2e-3
    assert_close(acc, ref, atol_frac=4e-3, rtol=3e-2)


def test_gemm_large_persistent():
    from rustorch_b200.ops import kernels as K_
    a, b = _mk((4096, 1024), 13), _mk((4096, 1024), 14)
    out = K_.gemm(a, b)
    assert rel_err(out, a.float() @ b.float().t()) < 1.5e-2


def test_fp16_linear_layer_runs_on_the_native_gemm():
    from rustorch_b200 import _native
    from rustorch_b200 import nn as rnn
    torch.manual_seed(0)
    lin = rnn.Linear(136, 72).cuda().half()
    x = torch.randn(5, 33, 136, device="cuda").half()
    x1, x2 = x.clone().requires_grad_(True), x.float().requires_grad_(True)
    n0 = _native.launch_count()
    y = lin(x1)
    assert _native.launch_count() > n0 and y.dtype == torch.float16
    ref = torch.nn.functional.linear(x2, lin.weight.detach().float(), lin.bias.detach().float())
    assert rel_err(y, ref) < 5e-3
    assert_close(y, ref, atol_frac=4e-3, rtol=3e-2)
    g = torch.randn_like(ref)
    y.backward(g.half())
    ref.backward(g.half().float())
    assert rel_err(x1.grad, x2.grad) < 5e-3
    assert_close(x1.grad, x2.grad, atol_frac=4e-3, rtol=3e-2)
    w32 = lin.weight.float().detach().requires_grad_(True)
    torch.nn.functional.linear(x.float(), w32, lin.bias.detach().float()).backward(g.half().float())
    assert rel_err(lin.weight.grad, w32.grad) < 5e-3
    assert_close(lin.weight.grad, w32.grad, atol_frac=4e-3, rtol=3e-2)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,Kd", [(256, 256, 64), (1000, 520, 200), (392, 2304, 768)])
def test_cta_pair_gemm_matches_fp32_reference(monkeypatch, M, N, Kd, a_mn, b_mn):
    """256 x 256 tiles over two CTAs (cta_group::2), forced on for every layout, ragged M / N / K tails included."""
    monkeypatch.setenv("RUSTORCH_GEMM_PAIR", "1")
    from rustorch_b200 import _native
    from rustorch_b200.ops import kernels as K
    torch.manual_seed(1)
    a = torch.randn((Kd, M) if a_mn else (M, Kd), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((Kd, N) if b_mn else (N, Kd), device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias)
    _native.check_status()
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    assert rel_err(out, af @ bf + bias.float()) < 1.5e-2


def test_cta_pair_gemm_split_k_and_batch(monkeypatch):
    monkeypatch.setenv("RUSTORCH_GEMM_PAIR", "1")
    from rustorch_b200.ops import kernels as K
    torch.manual_seed(2)
    a = torch.randn(8192, 512, device="cuda", dtype=torch.bfloat16)   # [K][M]
    b = torch.randn(8192, 768, device="cuda", dtype=torch.bfloat16)   # [K][N]
    acc = torch.zeros(512, 768, device="cuda")
    K.gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True, split_k=4)
    assert rel_err(acc, a.float().t() @ b.float()) < 2e-3
    x = torch.randn(3, 300, 256, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(3, 512, 256, device="cuda", dtype=torch.bfloat16)
    assert rel_err(K.gemm(x, w), x.float() @ w.float().transpose(1, 2)) < 1.5e-2


def test_fp32_linear_layer_runs_three_bf16_gemms_with_fp32_accuracy():
    from rustorch_b200 import _native
    from rustorch_b200 import nn as rnn
    torch.manual_seed(0)
    lin = rnn.Linear(264, 136).cuda()
    x = torch.randn(7, 19, 264, device="cuda")
    x1 = x.clone().requires_grad_(True)
    x2 = x.double().requires_grad_(True)
    n0 = _native.launch_count()
    y = lin(x1)
    assert _native.launch_count() >= n0 + 3 and y.dtype == torch.float32
    w64, b64 = lin.weight.detach().double().requires_grad_(True), lin.bias.detach().double()
    ref = torch.nn.functional.linear(x2, w64, b64)
    # split-bf16 keeps 16 mantissa bits per operand: far tighter than a tf32 product (~5e-4)
    torch.testing.assert_close(y.double(), ref, rtol=1e-4, atol=2e-4)
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.double())
    torch.testing.assert_close(x1.grad.double(), x2.grad, rtol=1e-4, atol=2e-4)
    torch.testing.assert_close(lin.weight.grad.double(), w64.grad, rtol=1e-4, atol=5e-4)
    torch.testing.assert_close(lin.bias.grad.double(), g.double().sum((0, 1)), rtol=1e-5, atol=1e-4)
