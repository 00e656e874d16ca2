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


def test_pruning_structures_schedules_and_wrapper():
    """Mask structures, the reference's schedule forms, lottery-ticket rewinding (src/nn/pruning.rs:30-640)."""
    torch.manual_seed(0)
    w = torch.randn(16, 8, 3, 3)
    # reference argument order: (method, structure, target_sparsity, schedule)
    ch = nn.Pruner(nn.PruningMethod.L2_NORM, nn.PruningStructure.CHANNEL, 0.25, nn.PruningSchedule.ONE_SHOT)
    out = ch.prune_tensor(w, "conv")
    dead = (out.flatten(1).abs().sum(1) == 0)
    assert int(dead.sum()) == 4                                      # whole output channels
    norms = w.flatten(1).norm(dim=1)
    assert set(dead.nonzero().flatten().tolist()) == set(norms.argsort()[:4].tolist())
    m = ch.get_mask("conv")
    assert m.pruned_count == 4 * 8 * 9 and m.remaining_params() == 12 * 8 * 9
    assert m.compression_ratio() == pytest.approx(1 / 0.75) and ch.get_global_sparsity() == pytest.approx(0.25)
    assert torch.equal(ch.reset_to_original_weights("conv"), w) and ch.reset_to_original_weights("x") is None
    fi = nn.Pruner(nn.PruningMethod.L1_NORM, nn.PruningStructure.FILTER, 0.5, nn.PruningSchedule.ONE_SHOT)
    assert int((fi.prune_tensor(w, "c").transpose(0, 1).flatten(1).abs().sum(1) == 0).sum()) == 4   # input channels
    # 2:4 blocks: exactly two survivors in every four consecutive weights, the two largest
    blk = nn.Pruner(nn.PruningMethod.L1_NORM, nn.PruningStructure.block(2, 4), 0.5, nn.PruningSchedule.ONE_SHOT)
    x = torch.randn(6, 10)                                           # 60 = 15 full blocks
    keep = blk.compute_mask(x)
    assert bool((keep.flatten().view(-1, 4).sum(1) == 2).all())
    top2 = x.abs().flatten().view(-1, 4).topk(2, dim=1).indices.sort(dim=1).values
    got = keep.flatten().view(-1, 4).nonzero()[:, 1].view(-1, 2)
    assert torch.equal(top2, got)
    rag = blk.compute_mask(torch.randn(7))                           # one block + a tail of 3 > n: 2 + 2 kept
    assert int(rag.sum()) == 4
    with pytest.raises(ValueError):
        nn.PruningStructure.block(3, 2)
    # schedules: zero before start, target after end, shaped in between
    for sched, mid in ((nn.PruningSchedule.linear(2, 6), 0.5), (nn.PruningSchedule.polynomial(2, 6, 3.0), 0.125),
                       (nn.PruningSchedule.exponential(2, 6), 1 - math.exp(-2.5))):
        p = nn.Pruner(nn.PruningMethod.L1_NORM, nn.PruningStructure.UNSTRUCTURED, 0.8, sched)
        assert p.current_sparsity() == 0.0
        for _ in range(4):
            p.step_epoch()
        assert p.current_sparsity() == pytest.approx(0.8 * mid)
        for _ in range(5):
            p.step_epoch()
        assert p.current_sparsity() == pytest.approx(0.8)
    # gradient / Taylor criteria use .grad when it is there
    lin = nn.Linear(8, 4)
    lin.weight.grad = torch.zeros_like(lin.weight)
    lin.weight.grad[0] = 1.0                                         # only row 0 matters to the loss
    g = nn.Pruner(nn.PruningMethod.GRADIENT, 0.75)
    g.prune(lin.named_parameters())
    assert bool((lin.weight[1:] == 0).all()) and bool((lin.weight[0] != 0).all())
    # wrapper: masks survive optimizer steps, rewind restores the surviving initial weights
    torch.manual_seed(1)
    net = nn.PruningAwareModule(nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 2)),
                                nn.Pruner(nn.PruningMethod.L1_NORM, 0.5))
    w0 = net.module[0].weight.detach().clone()
    net.enable_pruning()
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    for _ in range(3):
        opt.zero_grad()
        net(torch.randn(4, 8)).pow(2).mean().backward()
        opt.step()
    net(torch.randn(4, 8))                                           # forward re-applies the masks
    mask = net.pruner.masks["0.weight"]
    assert bool((net.module[0].weight[~mask] == 0).all()) and abs(net.get_statistics()["0.weight"] - 0.5) < 0.05
    net.pruner.rewind(net.module.named_parameters())
    assert torch.equal(net.module[0].weight.detach(), w0 * mask)
    net.pruner.clear_masks()
    assert net.pruner.get_global_sparsity() == 0.0


def test_quantizer_calibration_cache_and_qat():
    """Parameter objects, calibration modes, the per-layer cache and fake quantisation (src/nn/quantization.rs:22-447)."""
    p = nn.QuantizationParams.int8_symmetric(0.1)
    assert (p.qmin, p.qmax, p.zero_point, p.qtype) == (-128, 127, 0, nn.QuantizationType.INT8)
    qt = nn.QuantizedTensor(torch.tensor([10, 20, 30, -10, -20, -30], dtype=torch.int8), (2, 3), p)
    assert torch.allclose(qt.dequantize(), torch.tensor([[1., 2., 3.], [-1., -2., -3.]]), atol=1e-6)
    assert qt.compression_ratio() == 4.0 and qt.memory_bytes() == 6
    q = nn.Quantizer(nn.CalibrationMode.MIN_MAX, True)
    x = torch.tensor([1.0, 2.0, 3.0, -1.0, -2.0, -3.0]).view(2, 3)
    a = q.quantize_tensor(x, nn.QuantizationType.INT8, "layer")
    assert a.shape == (2, 3) and a.params.scale == pytest.approx(3 / 127) and int(a.data.max()) == 127
    b = q.quantize_tensor(10 * x, nn.QuantizationType.INT8, "layer")          # cached parameters are reused
    assert b.params is a.params and int(b.data.max()) == 127 and "layer" in q.get_statistics()
    q.clear_cache()
    assert q.quantize_tensor(10 * x, nn.QuantizationType.INT8, "layer").params.scale == pytest.approx(30 / 127)
    i4 = q.quantize_tensor(x, nn.QuantizationType.INT4)
    assert i4.params.qmax == 7 and i4.memory_bytes() == 3 and i4.compression_ratio() == 8.0
    h = q.quantize_tensor(x, nn.QuantizationType.FLOAT16)
    assert h.data.dtype == torch.float16 and torch.equal(h.dequantize(), x) and h.memory_bytes() == 12
    asym = nn.Quantizer(nn.CalibrationMode.MIN_MAX, False).quantize_tensor(torch.linspace(0, 1, 256), nn.QuantizationType.INT8)
    assert asym.params.zero_point == -128 and float((asym.dequantize() - torch.linspace(0, 1, 256)).abs().max()) < 2.1e-3
    # an outlier costs min / max calibration its resolution; percentile and entropy calibration clip it
    torch.manual_seed(0)
    y = torch.randn(20000)
    y[0] = 60.0
    body = y[1:]
    err = {}
    for name, mode in (("minmax", nn.CalibrationMode.MIN_MAX), ("pct", nn.CalibrationMode.percentile(0.999)),
                       ("kl", nn.CalibrationMode.ENTROPY)):
        t = nn.Quantizer(mode, True).quantize_tensor(y, nn.QuantizationType.INT8)
        err[name] = float((t.dequantize()[1:] - body).pow(2).mean())
    assert err["pct"] < 0.05 * err["minmax"] and err["kl"] < 0.25 * err["minmax"]
    assert len(nn.Quantizer().quantize_module(nn.Linear(4, 3), nn.QuantizationType.INT8, "fc")) == 2
    # quantisation-aware training: forward sees the grid, backward passes straight through inside the range
    qat = nn.QuantizationAwareModule(nn.Linear(4, 2), weights=True)
    xin = torch.tensor([[0.11, -0.52, 0.93, 2.0]], requires_grad=True)
    ref = qat(xin)
    assert torch.equal(ref, qat.module(xin))                                  # disabled: identity
    qat.set_qparams("input", nn.QuantizationParams.int8_symmetric(0.01))      # range +-1.27: 2.0 is clipped
    qat.enable_qat()
    fq = qat.apply_fake_quantization(xin, "input")
    assert torch.allclose(fq.detach(), torch.tensor([[0.11, -0.52, 0.93, 1.27]]), atol=1e-6)
    fq.sum().backward()
    assert torch.equal(xin.grad, torch.tensor([[1.0, 1.0, 1.0, 0.0]]))
    out = qat(xin)
    out.sum().backward()
    assert qat.module.weight.grad is not None and float((out - ref).abs().max()) > 0
    qat.set_fake_quantize(False)
    assert torch.equal(qat(xin), ref)
    obs = nn.QuantizationAwareModule(nn.Linear(4, 2))
    obs.enable_qat()
    obs.train()
    obs(torch.tensor([[1.0, -2.0, 0.5, 0.0]]))
    assert obs.qparams["input"].scale == pytest.approx(2.0 / 127)


def test_conv_validator_recurrent_helpers_and_stats():
    """src/nn/conv_base.rs:103-310, src/nn/recurrent_common.rs:13-450, src/nn/safe_ops.rs:236-270."""
    for bad in (dict(in_channels=0, out_channels=4, kernel_size=3), dict(in_channels=6, out_channels=4, kernel_size=3, groups=4),
                dict(in_channels=4, out_channels=4, kernel_size=0), dict(in_channels=4, out_channels=4, kernel_size=3, stride=0),
                dict(in_channels=4, out_channels=4, kernel_size=3, dilation=0), dict(in_channels=4, out_channels=4, kernel_size=3, groups=0)):
        with pytest.raises(ValueError):
            nn.Conv2d(**bad)
    with pytest.raises(ValueError):
        nn.MaxPool2d(0)
    with pytest.raises(ValueError):
        nn.AvgPool2d(2, stride=0)
    with pytest.raises(ValueError):
        nn.Validator.validate_adaptive_output_size((4, 0))
    assert nn.ConvOps.calc_output_size_1d(32, 3, 2, 1, 2) == 15
    assert nn.ConvOps.calc_output_size_2d((32, 28), (3, 5), (1, 2), (1, 2), (1, 1)) == (32, 14)
    assert nn.ConvOps.calc_output_size_3d((8, 16, 16), (3, 3, 3), (1, 2, 2), (1, 1, 1), (1, 1, 1)) == (8, 8, 8)
    c = nn.Conv3d(4, 6, 3, stride=(1, 2, 2), padding=1)
    assert tuple(c(torch.randn(1, 4, 8, 16, 16)).shape[2:]) == (8, 8, 8)
    assert nn.ConvOps.calc_transposed_output_size_1d(8, 3, 2, 1, 1) == nn.ConvTranspose1d(2, 2, 3, 2, 1, 1)(torch.randn(1, 2, 8)).shape[-1]
    w, b = nn.ConvOps.init_conv_params(8, 16, (3, 3), groups=2)
    assert w.shape == (16, 4, 3, 3) and b.shape == (16,) and float(b.abs().sum()) == 0 and w.requires_grad
    assert abs(float(w.std()) - math.sqrt(6 / 36)) < 0.05
    cfg = nn.RecurrentConfig.lstm(5, 7)
    assert (cfg.num_gates, cfg.gate_rows, nn.RecurrentConfig.gru(5, 7).num_gates, nn.RecurrentConfig.rnn(5, 7).num_gates) == (4, 28, 3, 1)
    w_ih, w_hh = nn.RecurrentOps.init_weights(cfg)
    b_ih, b_hh = nn.RecurrentOps.init_bias(cfg)
    assert w_ih.shape == (28, 5) and w_hh.shape == (28, 7) and float(w_ih.abs().max()) <= 1 / math.sqrt(7)
    assert float(b_ih[7:14].sum()) == 7.0 and float(b_ih.sum()) == 7.0 and float(b_hh.abs().sum()) == 0
    assert nn.RecurrentOps.init_bias(nn.RecurrentConfig.gru(5, 7, bias=False)) == (None, None)
    # one LSTM step from the helpers equals the cell
    cell = nn.LSTMCell(5, 7)
    x, h, cst = torch.randn(3, 5), torch.randn(3, 7), torch.randn(3, 7)
    gates = nn.RecurrentOps.add_variables(nn.RecurrentOps.linear_transform(x, cell.weight_ih, cell.bias_ih),
                                          nn.RecurrentOps.linear_transform(h, cell.weight_hh, cell.bias_hh))
    i, f, g, o = (nn.RecurrentOps.slice_gates(gates, k, 7) for k in range(4))
    c2 = nn.RecurrentOps.sigmoid(f) * cst + nn.RecurrentOps.sigmoid(i) * nn.RecurrentOps.tanh(g)
    h2 = nn.RecurrentOps.sigmoid(o) * nn.RecurrentOps.tanh(c2)
    hr, cr = cell(x, (h, cst))
    assert torch.allclose(h2, hr, atol=1e-6) and torch.allclose(c2, cr, atol=1e-6)
    with pytest.raises(IndexError):
        nn.RecurrentOps.slice_gates(gates, 4, 7)
    assert len(nn.collect_recurrent_parameters(w_ih, w_hh, b_ih, None)) == 3
    seq = torch.randn(2, 6, 5)
    assert torch.equal(nn.MultiLayerUtils.get_timestep_input(seq, 3, True), seq[:, 3])
    assert torch.equal(nn.MultiLayerUtils.get_timestep_input(seq.transpose(0, 1), 3, False), seq[:, 3])
    with pytest.raises(IndexError):
        nn.MultiLayerUtils.get_timestep_input(seq, 6, True)
    outs = [torch.randn(2, 7) for _ in range(6)]
    assert nn.MultiLayerUtils.stack_outputs(outs, True).shape == (2, 6, 7)
    assert nn.MultiLayerUtils.stack_outputs(outs, False).shape == (6, 2, 7)
    assert nn.MultiLayerUtils.stack_hidden_states(outs[:2]).shape == (2, 2, 7)
    assert nn.TrainingMode.TRAINING.is_training and not nn.TrainingMode.EVALUATION.is_training
    st = nn.SafeOps.get_stats(torch.tensor([1.0, 2.0, 3.0, 4.0]))
    assert (st.min, st.max, st.mean, st.count) == (1.0, 4.0, 2.5, 4) and st.variance == pytest.approx(1.25)
    assert st.std_dev() == pytest.approx(math.sqrt(1.25)) and st.is_reasonable() and st["std"] == st.std_dev()
    assert not nn.SafeOps.get_stats(torch.tensor([1.0, float("inf")])).is_reasonable()
    with pytest.raises(ValueError):
        nn.SafeOps.get_stats(torch.empty(0))
