"""CPU checks of the GPT model's PyTorch path, flat parameter store and fused-optimizer math."""
import torch

from rustorch_b200.models.gpt import GPT, GPTConfig
from rustorch_b200.optim.flat import FlatParams, FusedAdamW, FusedSGD


def _tiny():
    cfg = GPTConfig(vocab_size=97, n_positions=32, n_embd=32, n_layer=2, n_head=4, dropout=0.0)
    return cfg, GPT(cfg, seed=0)


def test_forward_shapes_and_loss():
    cfg, m = _tiny()
    idx = torch.randint(0, cfg.vocab_size, (3, 16))
    logits = m(idx)
    assert logits.shape == (3, 16, cfg.vocab_size)
    loss = m(idx, torch.roll(idx, -1, 1))
    assert abs(float(loss) - torch.log(torch.tensor(float(cfg.vocab_size)))) < 0.5


def test_defaults_match_reference_config():
    c = GPTConfig()
    assert (c.vocab_size, c.n_positions, c.n_embd, c.n_layer, c.n_head, c.dropout) == (50257, 1024, 768, 12, 12, 0.1)
    assert c.padded_vocab % 64 == 0 and c.padded_vocab >= c.vocab_size


def test_causality():
    cfg, m = _tiny()
    m.eval()
    idx = torch.randint(0, cfg.vocab_size, (1, 16))
    a = m(idx)
    idx2 = idx.clone()
    idx2[0, 10:] = (idx2[0, 10:] + 1) % cfg.vocab_size
    b = m(idx2)
    assert torch.allclose(a[0, :10], b[0, :10], atol=1e-5)


def test_flat_params_adamw_cpu_matches_torch():
    torch.manual_seed(0)
    lin = torch.nn.Linear(8, 4)
    ref = torch.nn.Linear(8, 4)
    ref.load_state_dict(lin.state_dict())
    flat = FlatParams(lin, decay_filter=lambda n, p: True)
    opt = FusedAdamW(flat, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for _ in range(3):
        gw, gb = torch.randn(4, 8), torch.randn(4)
        lin.weight.main_grad.copy_(gw.view(-1))
        lin.bias.main_grad.copy_(gb)
        ref.weight.grad, ref.bias.grad = gw.clone(), gb.clone()
        opt.step()
        ropt.step()
    assert torch.allclose(lin.weight, ref.weight, atol=1e-6)
    assert torch.allclose(lin.bias, ref.bias, atol=1e-6)
    assert float(flat.grad.abs().max()) == 0.0


def test_flat_params_groups_and_views():
    cfg, m = _tiny()
    flat = FlatParams(m)
    groups = flat.groups()
    assert groups[0][2] is True and groups[-1][2] is False
    views = flat.named_views(flat.master)
    assert views["blocks.0.w_qkv"].shape == (96, 32)
    for n, p, o, k in flat.entries:
        assert p.data_ptr() == flat.lp[o:o + k].data_ptr()
        assert o % 64 == 0


def test_fused_sgd_cpu():
    lin = torch.nn.Linear(4, 2)
    ref = torch.nn.Linear(4, 2)
    ref.load_state_dict(lin.state_dict())
    flat = FlatParams(lin)
    opt = FusedSGD(flat, lr=0.1, momentum=0.9, weight_decay=1e-3)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-3)
    for _ in range(3):
        gw, gb = torch.randn(2, 4), torch.randn(2)
        lin.weight.main_grad.copy_(gw.view(-1))
        lin.bias.main_grad.copy_(gb)
        ref.weight.grad, ref.bias.grad = gw.clone(), gb.clone()
        opt.step()
        ropt.step()
    assert torch.allclose(lin.weight, ref.weight, atol=1e-6)


def test_bench_reference_arm_reports_unavailable():
    import json
    import subprocess
    import sys
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line
