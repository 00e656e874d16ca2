"""Fused tensor-parallel GEMM kernels with a world of one rank (single GPU): the copy ring, the flag protocol
inside one device, tile ordering, staging and the reduce phase all run; peer traffic is covered by the multi-GPU test."""
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,K,N", [(128, 64, 128), (256, 512, 384), (1024, 1024, 1000), (384, 4096, 256)])
@pytest.mark.parametrize("b_mn", [False, True])
def test_all_gather_gemm_single_rank(rows, K, N, b_mn):
    from rustorch_b200 import _native
    from rustorch_b200.distributed.tp_fused import AllGatherGemm
    torch.manual_seed(0)
    op = AllGatherGemm(rows, K, "cuda")
    x = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    wt = w.t().contiguous() if b_mn else w
    for it in range(3):                                  # epochs advance; buffers are reused
        xi = (x * (it + 1)).bfloat16()
        y = op(wt, bias, x=xi, b_mn=b_mn)
        ref = xi.float() @ w.float().t() + bias.float()
        assert rel_err(y, ref) < 1e-2, it
        assert torch.equal(op.gather, xi)                # the gather buffer holds the full input afterwards
    _native.check_status()


@pytest.mark.parametrize("rows,K,N", [(128, 64, 128), (256, 512, 384), (1024, 1024, 1000), (256, 2048, 4096)])
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_reduce_scatter_single_rank(rows, K, N, b_mn):
    from rustorch_b200 import _native
    from rustorch_b200.distributed.tp_fused import GemmReduceScatter
    torch.manual_seed(1)
    op = GemmReduceScatter(rows, N, "cuda")
    x = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(rows, N, device="cuda").bfloat16()
    wt = w.t().contiguous() if b_mn else w
    for it in range(3):
        xi = (x * (it + 1)).bfloat16()
        y = op(xi, wt, bias, res, b_mn=b_mn)
        ref = xi.float() @ w.float().t() + bias.float() + res.float()
        assert rel_err(y, ref) < 1e-2, it
    _native.check_status()


def test_tp_linear_layers_forward_backward_single_rank():
    from rustorch_b200.distributed.tp_fused import FusedColumnParallelLinear, FusedRowParallelLinear
    torch.manual_seed(2)
    rows, d, ff = 256, 256, 1024
    col = FusedColumnParallelLinear(d, ff, rows)
    row = FusedRowParallelLinear(ff, d, rows)
    x = (torch.randn(rows, d, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    y = row(torch.nn.functional.gelu(col(x), approximate="tanh"))
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wc, bc, wr, br = (p.detach().float().requires_grad_(True) for p in (col.weight, col.bias, row.weight, row.bias))
    yr = torch.nn.functional.gelu(xr @ wc.t() + bc, approximate="tanh") @ wr.t() + br
    yr.backward(g.float())
    assert rel_err(y, yr) < 2e-2
    assert rel_err(x.grad, xr.grad) < 3e-2
    assert rel_err(col.weight.grad, wc.grad) < 3e-2 and rel_err(row.weight.grad, wr.grad) < 3e-2
    assert rel_err(col.bias.grad, bc.grad) < 3e-2 and rel_err(row.bias.grad, br.grad) < 3e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_p2p_collectives_single_rank(dtype):
    """World of one: flags and barriers still run; results equal the input."""
    from rustorch_b200 import _native
    from rustorch_b200.distributed.p2p_collectives import P2PCollectives
    pc = P2PCollectives(1 << 20, dtype, "cuda")
    x = torch.randn(1000, 33, device="cuda").to(dtype)
    for _ in range(3):
        assert torch.equal(pc.all_reduce(x), x)
    big = torch.randn(1 << 19, device="cuda").to(dtype)
    pc.one_shot_max_bytes = 0
    assert torch.equal(pc.all_reduce(big), big)
    assert torch.equal(pc.all_gather(x)[0], x)
    assert torch.equal(pc.reduce_scatter(big), big)
    y = x.clone()
    assert torch.equal(pc.broadcast(y), x) and int(pc.epoch_dev) == 7
    _native.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_allreduce_residual_norm_single_rank(dtype):
    """World of one: residual add + RMSNorm, call counter advances, receive slots untouched."""
    from rustorch_b200 import _native
    from rustorch_b200.distributed.p2p_collectives import AllReduceResidualNorm
    arn = AllReduceResidualNorm(16 * 4096, dtype, "cuda")
    w = (torch.rand(4096, device="cuda") + 0.5).to(dtype)
    for call, rows in enumerate((1, 16, 5)):
        part = torch.randn(rows, 4096, device="cuda").to(dtype)
        x = torch.randn(rows, 4096, device="cuda").to(dtype)
        x_ref = (x.float() + part.float()).to(dtype).float()
        h_ref = x_ref * torch.rsqrt(x_ref.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
        h = arn(part, x, w, 1e-6)
        assert torch.equal(x.float(), x_ref)
        assert float((h.float() - h_ref).abs().max() / h_ref.abs().max()) < 8e-3
        assert int(arn.state[0]) == call + 1
    assert not arn.fits(17, 4096) and arn.fits(16, 4096)
    _native.check_status()
