"""tcgen05 int8 GEMM (csrc/quant/gemm_i8_tcgen05.cu) against exact integer math, and the quantised ops built on it."""
import pytest
import torch

from rustorch_b200 import _native
from rustorch_b200 import quantization as Q

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 200, 272), (1, 8, 16), (513, 1000, 4096), (64, 129, 48)])
def test_int8_gemm_exact(M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randint(-128, 128, (M, K), device="cuda", generator=g, dtype=torch.int8)
    b = torch.randint(-128, 128, (N, K), device="cuda", generator=g, dtype=torch.int8)
    n0 = _native.launch_count()
    acc = Q.int8_gemm(a, b)
    assert _native.launch_count() == n0 + 1
    want = (a.double() @ b.double().t()).to(torch.int32)       # exact: |sum| < 2^53
    assert acc.dtype == torch.int32 and torch.equal(acc, want)


def test_int8_gemm_fused_dequant_epilogue_and_ragged_k():
    g = torch.Generator(device="cuda").manual_seed(5)
    M, N, K = 200, 136, 100                                     # K not a multiple of 16: zero padded inside
    a = torch.randint(-128, 128, (M, K), device="cuda", generator=g, dtype=torch.int8)
    b = torch.randint(-128, 128, (N, K), device="cuda", generator=g, dtype=torch.int8)
    rs = torch.rand(M, device="cuda", generator=g) * 0.1
    cs = torch.rand(N, device="cuda", generator=g) * 0.1
    bias = torch.randn(N, device="cuda", generator=g)
    want = (a.double() @ b.double().t()) * rs.double()[:, None] * cs.double()[None, :] + bias.double()
    torch.testing.assert_close(Q.int8_gemm(a, b, rs, cs, bias).double(), want, rtol=1e-5, atol=1e-4)
    want1 = (a.double() @ b.double().t()) * 0.5 * 0.25
    torch.testing.assert_close(Q.int8_gemm(a, b, torch.tensor([0.5]), torch.tensor([0.25])).double(), want1, rtol=1e-6, atol=1e-4)


def test_quantised_ops_run_on_the_native_gemm():
    torch.manual_seed(0)
    x = torch.randn(70, 96, device="cuda")
    w = torch.randn(48, 96, device="cuda") * 0.2
    qx = Q.quantize(x, torch.tensor(0.03, device="cuda"), torch.tensor(0, device="cuda"), Q.QuantizationType.INT8)
    sw = w.abs().amax(1) / 127.0
    qw = Q.QuantizedTensor((w / sw[:, None]).round().clamp(-127, 127).to(torch.int8), sw, torch.zeros(48, dtype=torch.int32, device="cuda"),
                           Q.QuantizationType.INT8, 0)
    n0 = _native.launch_count()
    y = Q.qlinear(qx, qw, torch.ones(48, device="cuda"))
    assert _native.launch_count() > n0
    ref = qx.dequantize() @ qw.dequantize().t() + 1.0
    torch.testing.assert_close(y, ref, rtol=1e-3, atol=1e-3)
    # qmatmul_cuda: per-tensor operands with zero points
    a = Q.quantize(x, torch.tensor(0.05, device="cuda"), torch.tensor(3, device="cuda"), Q.QuantizationType.INT8)
    bt = Q.quantize(w.t().contiguous(), torch.tensor(0.01, device="cuda"), torch.tensor(-2, device="cuda"), Q.QuantizationType.INT8)
    n0 = _native.launch_count()
    out = Q.qmatmul_cuda(a, bt)
    assert _native.launch_count() > n0
    ref = a.dequantize() @ bt.dequantize()
    assert (out.dequantize() - ref).abs().max() <= 2 * float(out.scale)
    # qconv2d_cuda: unfolded patches through the same kernel
    img = torch.randn(2, 8, 12, 12, device="cuda")
    filt = torch.randn(16, 8, 3, 3, device="cuda") * 0.2
    qi = Q.quantize(img, torch.tensor(0.04, device="cuda"), torch.tensor(1, device="cuda"), Q.QuantizationType.INT8)
    qf = Q.quantize(filt, torch.tensor(0.01, device="cuda"), torch.tensor(0, device="cuda"), Q.QuantizationType.INT8)
    n0 = _native.launch_count()
    yc = Q.qconv2d_cuda(qi, qf, torch.zeros(16, device="cuda"), stride=2, padding=1)
    assert _native.launch_count() > n0
    refc = torch.nn.functional.conv2d(qi.dequantize(), qf.dequantize(), None, 2, 1)
    torch.testing.assert_close(yc, refc, rtol=1e-3, atol=1e-3)
