"""Norm / embedding / cross-entropy / optimizer / reduction kernels vs fp32 PyTorch."""
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _bf(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("rows,C", [(64, 768), (1000, 256), (33, 4096), (700, 2048), (50, 8192), (40, 3072)])
def test_layer_norm_fwd_bwd(rows, C):
    from rustorch_b200.ops import kernels as K_
    x, w, b, dy, dres = _bf((rows, C), 1), _bf((C,), 2), _bf((C,), 3), _bf((rows, C), 4), _bf((rows, C), 5)
    y, mean, rstd = K_.layer_norm_fwd(x, w, b, 1e-5)
    xr = x.float().requires_grad_(True)
    wr, br = w.float().requires_grad_(True), b.float().requires_grad_(True)
    yr = F.layer_norm(xr, (C,), wr, br, 1e-5)
    assert rel_err(y, yr) < 1e-2
    yr.backward(dy.float())
    dg = torch.zeros(C, device="cuda")
    db = torch.zeros(C, device="cuda")
    dx = K_.layer_norm_bwd(dy, x, w, mean, rstd, dg, db, dres=dres)
    assert rel_err(dx, xr.grad + dres.float()) < 1.5e-2
    assert rel_err(dg, wr.grad) < 1e-2
    assert rel_err(db, br.grad) < 1e-2


@pytest.mark.parametrize("rows,C", [(128, 512), (77, 4096), (1300, 4096), (19, 8192), (64, 5120)])
def test_rms_norm_fwd_bwd(rows, C):
    from rustorch_b200.ops import kernels as K_
    x, w, dy = _bf((rows, C), 1), _bf((C,), 2), _bf((rows, C), 4)
    eps = 1e-5
    y, rstd = K_.rms_norm_fwd(x, w, eps)
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + eps) * wr
    assert rel_err(y, yr) < 1e-2
    yr.backward(dy.float())
    dg = torch.zeros(C, device="cuda")
    dx = K_.rms_norm_bwd(dy, x, w, rstd, dg)
    assert rel_err(dx, xr.grad) < 1.5e-2
    assert rel_err(dg, wr.grad) < 1e-2


def test_embedding_fwd_bwd():
    from rustorch_b200.ops import kernels as K_
    V, T, C, B = 1000, 64, 256, 4
    wte, wpe = _bf((V, C), 1), _bf((T, C), 2)
    idx = torch.randint(0, V, (B, T), device="cuda")
    out = K_.embedding_fwd(idx, wte, wpe, T)
    ref = wte.float()[idx] + wpe.float()[None]
    assert rel_err(out, ref) < 1e-2
    dout = _bf((B, T, C), 3)
    dwte = torch.zeros(V, C, device="cuda")
    dwpe = torch.zeros(T, C, device="cuda")
    K_.embedding_bwd(idx, dout, dwte, dwpe, T, V)
    ref_wte = torch.zeros(V, C, device="cuda").index_add_(0, idx.view(-1), dout.float().view(-1, C))
    assert rel_err(dwte, ref_wte) < 1e-4
    assert rel_err(dwpe, dout.float().sum(0)) < 1e-4


@pytest.mark.parametrize("rows,vocab,ld", [(64, 1000, 1024), (16, 50257, 50304), (8, 70000, 70016)])
def test_cross_entropy_fused(rows, vocab, ld):
    from rustorch_b200.ops import kernels as K_
    logits = _bf((rows, ld), 1, scale=2.0)
    tgt = torch.randint(0, vocab, (rows,), device="cuda")
    lr = logits[:, :vocab].float().requires_grad_(True)
    ref = F.cross_entropy(lr, tgt, reduction="sum")
    ref.backward()
    work = logits.clone()
    loss = K_.cross_entropy_(work, tgt, vocab, 1.0)
    assert abs(float(loss.sum()) - float(ref)) / abs(float(ref)) < 2e-3
    assert rel_err(work[:, :vocab], lr.grad) < 1e-2
    assert float(work[:, vocab:].abs().max()) == 0.0 if ld > vocab else True


def test_colsum_and_reduce():
    from rustorch_b200.ops import kernels as K_
    x = _bf((1000, 770), 1)
    out = torch.ones(770, device="cuda")
    K_.colsum_accum(x, out)
    assert rel_err(out, 1 + x.float().sum(0)) < 1e-4
    f = torch.randn(1 << 20, device="cuda")
    assert abs(float(K_.reduce_all(f, "sum")) - float(f.double().sum())) < 1.0
    assert abs(float(K_.reduce_all(f, "sumsq")) - float(f.double().pow(2).sum())) / (1 << 20) < 1e-3
    assert float(K_.reduce_all(f, "max")) == float(f.max())
    assert float(K_.reduce_all(f, "min")) == float(f.min())


@pytest.mark.parametrize("decoupled", [True, False])
def test_fused_adamw_matches_torch(decoupled):
    from rustorch_b200.optim.flat import FlatParams, FusedAdamW
    torch.manual_seed(0)
    lin = torch.nn.Linear(64, 48).cuda().to(torch.bfloat16)
    ref = torch.nn.Linear(64, 48).cuda()
    ref.load_state_dict({k: v.float() for k, v in lin.state_dict().items()})
    flat = FlatParams(lin, decay_filter=lambda n, p: True)
    opt = FusedAdamW(flat, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, decoupled=decoupled)
    cls = torch.optim.AdamW if decoupled else torch.optim.Adam
    ropt = cls(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(5):
        gw = torch.randn(48, 64, device="cuda")
        gb = torch.randn(48, device="cuda")
        lin.weight.main_grad.copy_(gw.view(-1))
        lin.bias.main_grad.copy_(gb)
        ref.weight.grad, ref.bias.grad = gw.clone(), gb.clone()
        opt.step()
        ropt.step()
    views = flat.named_views(flat.master)
    assert rel_err(views["weight"], ref.weight) < 1e-5
    assert rel_err(views["bias"], ref.bias) < 1e-5
    assert float(flat.grad.abs().max()) == 0.0
    assert rel_err(lin.weight, ref.weight) < 1e-2


def test_fused_sgd_momentum_matches_torch():
    from rustorch_b200.optim.flat import FlatParams, FusedSGD
    torch.manual_seed(0)
    lin = torch.nn.Linear(32, 16).cuda().to(torch.bfloat16)
    ref = torch.nn.Linear(32, 16).cuda()
    ref.load_state_dict({k: v.float() for k, v in lin.state_dict().items()})
    flat = FlatParams(lin)
    opt = FusedSGD(flat, lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=True)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=True)
    for _ in range(4):
        gw, gb = torch.randn(16, 32, device="cuda"), torch.randn(16, device="cuda")
        lin.weight.main_grad.copy_(gw.view(-1))
        lin.bias.main_grad.copy_(gb)
        ref.weight.grad, ref.bias.grad = gw.clone(), gb.clone()
        opt.step()
        ropt.step()
    views = flat.named_views(flat.master)
    assert rel_err(views["weight"], ref.weight) < 1e-5


def test_ddp_bucket_kernel_single_rank_matches_fused_adamw():
    """world = 1: the bucket kernel is a fused AdamW over buckets and must equal FusedAdamW."""
    from rustorch_b200.distributed.fused_allreduce import FusedDDPAdamW
    from rustorch_b200.optim.flat import FlatParams, FusedAdamW
    from rustorch_b200.nn import fused
    torch.manual_seed(0)
    a = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.Linear(512, 128)).cuda().to(torch.bfloat16)
    b = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.Linear(512, 128)).cuda().to(torch.bfloat16)
    b.load_state_dict(a.state_dict())
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ddp = FusedDDPAdamW(a, bucket_cap_mb=0.25, overlap=False, **hp)
    flat = FlatParams(b)
    opt = FusedAdamW(flat, **hp)
    assert ddp.n_buckets > 2
    for _ in range(3):
        g = torch.randn(flat.numel, device="cuda")
        ddp.flat.grad.copy_(g)
        flat.grad.copy_(g)
        ddp.step()
        opt.step()
    torch.cuda.synchronize()
    assert float((ddp.flat.master - flat.master).abs().max()) < 1e-6
    assert float((ddp.flat.lp.float() - flat.lp.float()).abs().max()) == 0.0
    assert float(ddp.flat.grad.abs().max()) == 0.0
    ddp.close()
    assert fused.grad_ready_hook is None
