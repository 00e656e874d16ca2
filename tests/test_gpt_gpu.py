"""End-to-end: fused GPT forward/backward/step on the native kernels vs the PyTorch restatement."""
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _models():
    from rustorch_b200.models.gpt import GPT, GPTConfig
    cfg = GPTConfig(vocab_size=1000, n_positions=256, n_embd=256, n_layer=2, n_head=4, dropout=0.0)
    m = GPT(cfg, device="cuda", dtype=torch.bfloat16, seed=0)
    ref = GPT(cfg, device="cuda", dtype=torch.float32, seed=0)
    return cfg, m, ref


def test_gpt_loss_and_grads_match_reference():
    from rustorch_b200.optim.flat import FlatParams
    cfg, m, ref = _models()
    flat = FlatParams(m)
    g = torch.Generator(device="cuda").manual_seed(0)
    idx = torch.randint(0, cfg.vocab_size, (4, 256), device="cuda", generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (4, 256), device="cuda", generator=g)
    loss = m(idx, tgt)
    loss.backward()
    rloss = ref(idx, tgt)
    rloss.backward()
    assert abs(float(loss) - float(rloss)) / float(rloss) < 1e-2
    grads = flat.named_views(flat.grad)
    refg = dict(ref.named_parameters())
    for name in ["blocks.0.w_qkv", "blocks.1.w_fc2", "blocks.0.b_fc", "blocks.1.ln1_w", "lnf_b", "wpe",
                 "lm_head", "wte", "blocks.0.w_proj", "blocks.1.b_qkv"]:
        assert rel_err(grads[name], refg[name].grad) < 6e-2, name


def test_gpt_training_reduces_loss():
    from rustorch_b200.optim.flat import FlatParams, FusedAdamW
    cfg, m, _ = _models()
    flat = FlatParams(m)
    opt = FusedAdamW(flat, lr=3e-3, betas=(0.9, 0.95), weight_decay=0.1)
    g = torch.Generator(device="cuda").manual_seed(1)
    idx = torch.randint(0, cfg.vocab_size, (4, 256), device="cuda", generator=g)
    tgt = torch.roll(idx, -1, 1)
    losses = []
    for _ in range(12):
        loss = m(idx, tgt)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0] - 1.0, losses


def test_gpt_inference_logits():
    cfg, m, ref = _models()
    idx = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda")
    with torch.no_grad():
        out = m(idx)
        r = ref(idx)
    assert out.shape == r.shape
    assert rel_err(out, r) < 5e-2


def _grads_of(m, flat, idx, tgt, loss_fn):
    flat.grad.zero_()
    loss = m(idx, tgt)
    loss_fn(loss).backward()
    return float(loss), {k: v.clone() for k, v in flat.named_views(flat.grad).items()}


def test_lm_head_loss_applies_upstream_gradient():
    """(2 * loss).backward() doubles every gradient: the fused loss reads the upstream factor on the device."""
    from rustorch_b200.optim.flat import FlatParams
    cfg, m, ref = _models()
    flat = FlatParams(m)
    g = torch.Generator(device="cuda").manual_seed(3)
    idx = torch.randint(0, cfg.vocab_size, (2, 256), device="cuda", generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, 256), device="cuda", generator=g)
    (ref(idx, tgt) * 2.0).backward()
    refg = dict(ref.named_parameters())
    _, g2 = _grads_of(m, flat, idx, tgt, lambda l: l * 2.0)
    for name in ["lm_head", "lnf_w", "blocks.1.w_fc2", "blocks.0.w_qkv", "wte"]:
        assert rel_err(g2[name], refg[name].grad) < 6e-2, name
    # a loss scaler: scale by 65536, unscale the gradients, compare with the unscaled oracle
    _, gs = _grads_of(m, flat, idx, tgt, lambda l: l * 65536.0)
    for name in ["lm_head", "blocks.0.w_qkv"]:
        assert rel_err(gs[name] / 65536.0, refg[name].grad / 2.0) < 6e-2, name


def test_lm_head_loss_ignore_index_matches_reference_mean():
    """Rows equal to ignore_index are left out of the mean, as in F.cross_entropy."""
    from rustorch_b200.optim.flat import FlatParams
    cfg, m, ref = _models()
    flat = FlatParams(m)
    g = torch.Generator(device="cuda").manual_seed(4)
    idx = torch.randint(0, cfg.vocab_size, (2, 256), device="cuda", generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, 256), device="cuda", generator=g)
    tgt[:, 100:] = -100                       # 61 % of the rows are padding
    rloss = ref(idx, tgt)
    rloss.backward()
    refg = dict(ref.named_parameters())
    loss, grads = _grads_of(m, flat, idx, tgt, lambda l: l)
    assert abs(loss - float(rloss)) / float(rloss) < 1e-2
    for name in ["lm_head", "lnf_w", "blocks.0.w_qkv"]:
        assert rel_err(grads[name], refg[name].grad) < 6e-2, name


def test_gpt_fused_path_with_dropout_trains_and_masks_are_replayed():
    """dropout > 0 runs on the fused path: training reduces the loss, eval is deterministic, and with the same seed
    two forward + backward passes give identical gradients (the backward pass regenerates the forward masks)."""
    from rustorch_b200.models.gpt import GPT, GPTConfig
    from rustorch_b200.optim.flat import FlatParams, FusedAdamW
    from rustorch_b200.ops import pool
    cfg = GPTConfig(vocab_size=1000, n_positions=256, n_embd=256, n_layer=2, n_head=4, dropout=0.1)
    m = GPT(cfg, device="cuda", dtype=torch.bfloat16, seed=0)
    flat = FlatParams(m)
    opt = FusedAdamW(flat, lr=3e-3, betas=(0.9, 0.95), weight_decay=0.1)
    g = torch.Generator(device="cuda").manual_seed(1)
    idx = torch.randint(0, cfg.vocab_size, (4, 256), device="cuda", generator=g)
    tgt = torch.roll(idx, -1, 1)
    m.train()

    def grads_with_seed(seed):
        torch.manual_seed(seed)
        pool._offsets.clear()
        flat.grad.zero_()
        loss = m(idx, tgt)
        loss.backward()
        return float(loss), flat.grad.clone()
    l1, g1 = grads_with_seed(5)
    l2, g2 = grads_with_seed(5)
    l3, g3 = grads_with_seed(6)
    assert l1 == l2 and torch.allclose(g1, g2, rtol=1e-3, atol=1e-5)      # fp32 atomics reorder sums only
    assert l3 != l1
    flat.grad.zero_()
    losses = []
    for _ in range(12):
        loss = m(idx, tgt)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0] - 1.0, losses
    m.eval()
    with torch.no_grad():
        a, b = m(idx), m(idx)
    assert torch.equal(a, b)
