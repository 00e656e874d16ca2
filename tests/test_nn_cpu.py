"""nn layer surface and semantics on CPU."""
import math

import pytest
import torch

from rustorch_b200 import nn


def test_linear_init_and_shapes():
    torch.manual_seed(0)
    l = nn.Linear(512, 256)
    assert l.weight.shape == (256, 512) and l.bias.shape == (256,)
    assert abs(float(l.weight.std()) - math.sqrt(2 / 512)) < 5e-3
    assert abs(float(l.bias.std()) - math.sqrt(2 / 512)) < 2e-2      # bias is N(0, sqrt(2/in)) too
    assert nn.Linear.new_no_bias(8, 4).bias is None
    assert l(torch.randn(2, 3, 512)).shape == (2, 3, 256)


def test_conv_family_shapes_and_grads():
    c2 = nn.Conv2d(3, 8, (3, 3), stride=(2, 2), padding=(1, 1))
    x = torch.randn(2, 3, 16, 16, requires_grad=True)
    y = c2(x)
    assert y.shape == (2, 8, 8, 8) and c2.output_size(16, 16) == (8, 8)
    y.sum().backward()
    assert x.grad is not None and c2.weight.grad is not None
    assert nn.Conv1d(4, 6, 3, padding=1)(torch.randn(2, 4, 10)).shape == (2, 6, 10)
    assert nn.Conv3d(2, 4, (3, 3, 3), 1, 1, 1, 2)(torch.randn(1, 2, 5, 5, 5)).shape == (1, 4, 5, 5, 5)
    assert nn.ConvTranspose2d.upsample_2x(4)(torch.randn(1, 4, 8, 8)).shape == (1, 4, 16, 16)
    assert nn.ConvTranspose1d(4, 2, 3, stride=2, output_padding=1)(torch.randn(1, 4, 5)).shape == (1, 2, 12)


def test_norm_layers():
    bn = nn.BatchNorm2d(4)
    x = torch.randn(8, 4, 5, 5) * 3 + 1
    y = bn(x)
    assert abs(float(y.mean())) < 1e-4 and bn.is_training()
    assert float(bn.get_running_mean().abs().sum()) > 0
    bn.eval()
    assert not bn.is_training()
    ln = nn.LayerNorm([16])
    assert torch.allclose(ln(torch.randn(3, 16)).mean(-1), torch.zeros(3), atol=1e-5)
    r = nn.RMSNorm(16)
    assert r.eps == 1e-8
    xr = torch.randn(3, 16)
    assert torch.allclose(r(xr), xr / xr.pow(2).mean(-1, keepdim=True).sqrt(), atol=1e-4)
    assert nn.GroupNorm(2, 4)(torch.randn(2, 4, 3, 3)).shape == (2, 4, 3, 3)
    assert nn.InstanceNorm2d(4)(torch.randn(2, 4, 3, 3)).shape == (2, 4, 3, 3)


def test_activations_and_dropout():
    x = torch.tensor([-1.0, 0.0, 2.0])
    assert torch.allclose(nn.gelu(x), torch.nn.functional.gelu(x, approximate="tanh"))
    assert torch.allclose(nn.swiglu(torch.tensor([1.0, 2.0, 3.0, 4.0])),
                          torch.nn.functional.silu(torch.tensor([1.0, 2.0])) * torch.tensor([3.0, 4.0]))
    assert torch.allclose(nn.softmax(torch.zeros(2, 4)).sum(-1), torch.ones(2))
    d = nn.Dropout(0.5)
    d.eval()
    assert torch.equal(d(x), x)
    d.train()
    out = d(torch.ones(10000))
    assert abs(float(out.mean()) - 1.0) < 0.05 and set(out.unique().tolist()) <= {0.0, 2.0}
    with pytest.raises(ValueError):
        nn.Dropout(1.5)


def test_embedding_and_positional():
    e = nn.Embedding(10, 4, padding_idx=0, freeze=True)
    assert not e.weight.requires_grad and float(e.weight[0].abs().sum()) == 0
    assert e(torch.tensor([[1, 2, 0]])).shape == (1, 3, 4)
    pe = nn.PositionalEmbedding(16, 4)
    assert pe(torch.zeros(2, 8, 4)).shape == (2, 8, 4)
    with pytest.raises(ValueError):
        pe(torch.zeros(1, 32, 4))
    s = nn.SinusoidalPositionalEncoding(16, 4)(torch.zeros(1, 3, 4))
    assert torch.allclose(s[0, 0], torch.tensor([0.0, 1.0, 0.0, 1.0]))
    assert nn.PositionalEncoding(8)(torch.zeros(1, 5, 8)).shape == (1, 5, 8)


def test_multihead_attention_matches_torch():
    torch.manual_seed(0)
    m = nn.MultiheadAttention(32, 4)
    ref = torch.nn.MultiheadAttention(32, 4, batch_first=True)
    with torch.no_grad():
        ref.in_proj_weight.copy_(m.in_proj.weight)
        ref.in_proj_bias.copy_(m.in_proj.bias)
        ref.out_proj.weight.copy_(m.out_proj.weight)
        ref.out_proj.bias.copy_(m.out_proj.bias)
    x = torch.randn(2, 6, 32)
    out, w = m(x, x, x)
    ro, rw = ref(x, x, x)
    assert torch.allclose(out, ro, atol=1e-5) and torch.allclose(w, rw, atol=1e-5)
    assert torch.allclose(w.sum(-1), torch.ones(2, 6), atol=1e-5)          # per-row softmax
    mask = torch.ones(6, 6).tril()
    out_c, w_c = m(x, x, x, attn_mask=mask)
    assert float(w_c[0].triu(1).abs().max()) < 1e-6
    out_c2, _ = m(x, x, x, need_weights=False, is_causal=True)
    assert torch.allclose(out_c, out_c2, atol=1e-5)
    kpm = torch.ones(2, 6)
    kpm[:, -2:] = 0
    _, w_k = m(x, x, x, key_padding_mask=kpm)
    assert float(w_k[..., -2:].abs().max()) < 1e-6


def test_transformer_stack_and_rnn():
    t = nn.Transformer(d_model=32, nhead=4, num_encoder_layers=2, num_decoder_layers=2, dim_feedforward=64, dropout=0.0)
    src, tgt = torch.randn(2, 5, 32), torch.randn(2, 3, 32)
    out = t(src, tgt, tgt_mask=nn.Transformer.generate_square_subsequent_mask(3))
    assert out.shape == (2, 3, 32)
    out.sum().backward()
    enc = nn.TransformerEncoderLayer(32, 4, 64, 0.0, "gelu", norm_first=True)
    assert enc(src, is_causal=True).shape == (2, 5, 32)
    lstm = nn.LSTM(8, 16, 2, True, True, 0.0, True)
    y, (h, c) = lstm(torch.randn(3, 7, 8))
    assert y.shape == (3, 7, 32) and h.shape == (4, 3, 16)
    hc = nn.LSTMCell(8, 16)(torch.randn(3, 8))
    assert hc[0].shape == (3, 16)
    assert nn.GRU(8, 16)(torch.randn(7, 3, 8))[0].shape == (7, 3, 16)
    assert nn.RNN(8, 16)(torch.randn(7, 3, 8))[0].shape == (7, 3, 16)


def test_losses():
    logits = torch.randn(5, 7, requires_grad=True)
    tgt = torch.randint(0, 7, (5,))
    l = nn.CrossEntropyLoss()(logits, tgt)
    assert torch.allclose(l, torch.nn.functional.cross_entropy(logits, tgt))
    l.backward()
    assert nn.MSELoss("sum")(torch.ones(3), torch.zeros(3)).item() == 3.0
    assert nn.FocalLoss(1.0, 0.0)(logits, tgt).item() == pytest.approx(l.item(), rel=1e-5)
    a, p, n = torch.randn(4, 8), torch.randn(4, 8), torch.randn(4, 8)
    assert nn.TripletMarginLoss()(a, p, n).item() >= 0
    assert nn.BCEWithLogitsLoss()(torch.zeros(4), torch.ones(4)).item() == pytest.approx(math.log(2), rel=1e-5)
    assert nn.MarginRankingLoss(0.5)(torch.ones(3), torch.zeros(3), torch.ones(3)).item() == 0.0
    assert nn.KLDivLoss("sum")(torch.log(torch.tensor([0.5, 0.5])), torch.tensor([0.5, 0.5])).item() == pytest.approx(0.0, abs=1e-6)
    assert nn.CosineEmbeddingLoss()(a, a, torch.ones(4)).item() == pytest.approx(0.0, abs=1e-6)


def test_pruning_quantization_safeops():
    lin = nn.Linear(32, 16)
    pr = nn.Pruner(nn.PruningMethod.MAGNITUDE, 0.5)
    rep = pr.prune(lin.named_parameters())
    assert abs(rep["weight"] - 0.5) < 0.02 and float((lin.weight == 0).float().mean()) > 0.45
    g = nn.Pruner(nn.PruningMethod.STRUCTURED, 0.25, nn.PruningSchedule.GRADUAL, total_steps=2)
    g.prune(lin.named_parameters())
    assert g.current_sparsity() == pytest.approx(0.125)
    q = nn.Quantizer(nn.QuantizationType.INT8_ASYMMETRIC)
    x = torch.randn(100)
    qt = q.quantize(x)
    assert qt.data.dtype == torch.int8 and float((qt.dequantize() - x).abs().max()) < 0.05
    assert nn.Quantizer(nn.QuantizationType.INT4_SYMMETRIC).quantize(x).data.abs().max() <= 7
    with pytest.raises(ValueError):
        nn.SafeOps.create_variable([1.0, float("nan")], [2])
    assert nn.SafeOps.get_stats(torch.ones(4))["mean"] == 1.0
    s = nn.Sequential(nn.Linear(4, 4), nn.ReLU()).add(nn.Linear(4, 2))
    assert s.len() == 3 and s(torch.randn(1, 4)).shape == (1, 2)
