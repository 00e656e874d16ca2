"""CPU tests: vision, visualization, quantization."""
import gzip
import os

import numpy as np
import pytest
import torch

from rustorch_b200 import quantization as Q, vision as V, visualization as Z


# ------------------------------------------------------------------ vision
def test_transforms_shapes_and_values():
    img = torch.arange(3 * 8 * 10, dtype=torch.float32).reshape(3, 8, 10)
    assert V.Resize((4, 5))(img).shape == (3, 4, 5)
    assert V.Resize(16, V.InterpolationMode.NEAREST)(img.unsqueeze(0)).shape == (1, 3, 16, 16)
    assert torch.equal(V.CenterCrop(4)(img), img[:, 2:6, 3:7])
    g = torch.Generator().manual_seed(0)
    assert V.RandomCrop(6, padding=2, generator=g)(img).shape == (3, 6, 6)
    assert torch.equal(V.RandomHorizontalFlip(1.0)(img), img.flip(-1)) and torch.equal(V.RandomHorizontalFlip(0.0)(img), img)
    batch = torch.stack([img, img + 1])
    fl = V.RandomHorizontalFlip(0.5, torch.Generator().manual_seed(1))(batch)
    assert fl.shape == batch.shape
    n = V.Normalize([1.0, 2.0, 3.0], [2.0, 2.0, 2.0])(torch.ones(3, 2, 2) * 3)
    assert torch.allclose(n[:, 0, 0], torch.tensor([1.0, 0.5, 0.0]))
    hwc = (np.arange(2 * 3 * 3) % 255).astype(np.uint8).reshape(2, 3, 3)
    t = V.ToTensor()(hwc)
    assert t.shape == (3, 2, 3) and t.max() <= 1.0
    rot = V.RandomRotation(0.0)(torch.rand(1, 9, 9))
    assert rot.shape == (1, 9, 9)
    with pytest.raises(ValueError):
        V.CenterCrop(20)(img)
    im = V.Image(torch.zeros(4, 5, 3), V.ImageFormat.HWC)
    assert (im.height, im.width, im.channels) == (4, 5, 3) and im.to_chw().data.shape == (3, 4, 5)


def test_pipeline_builder_stats_cache_and_presets():
    p = (V.PipelineBuilder("p").transform(V.Resize(8)).conditional(V.CenterCrop(4), lambda x: x.shape[-1] > 4)
         .transform(V.Normalize([0.5], [0.5])).cache(2).build())
    x = torch.rand(1, 16, 16)
    y = p(x, key="a")
    assert y.shape == (1, 4, 4) and p(x, key="a") is y and p.stats.cache_hits == 1 and p.stats.total_processed == 1
    assert set(p.stats.per_transform_s) == {"Resize", "if:CenterCrop", "Normalize"}
    val = V.ImageNetPreprocessing.validation()
    out = val(torch.randint(0, 255, (3, 300, 280), dtype=torch.uint8).float())
    assert out.shape == (3, 224, 224)
    assert V.CIFARPreprocessing.training()(torch.rand(3, 32, 32)).shape == (3, 32, 32)
    pb = V.PipelineBuilder().transform(V.Resize(4)).execution_mode(V.ExecutionMode.BATCH).build()
    outs = pb.process_batch([torch.rand(1, 8, 8) for _ in range(3)])
    assert len(outs) == 3 and outs[0].shape == (1, 4, 4)


def test_datasets_read_standard_files(tmp_path):
    imgs = (np.random.rand(5, 28, 28) * 255).astype(np.uint8)
    labels = np.array([3, 1, 4, 1, 5], dtype=np.uint8)
    V.write_idx(str(tmp_path / "train-images-idx3-ubyte.gz"), imgs)
    V.write_idx(str(tmp_path / "train-labels-idx1-ubyte"), labels)
    ds = V.MNIST(str(tmp_path), train=True)
    x, y = ds[2]
    assert len(ds) == 5 and x.shape == (1, 28, 28) and y == 4 and torch.allclose(x[0], torch.from_numpy(imgs[2]).float() / 255)
    rec = np.zeros((4, 3073), dtype=np.uint8)
    rec[:, 0] = [9, 0, 1, 2]
    rec[:, 1:] = np.random.randint(0, 255, (4, 3072))
    for i in range(1, 6):
        rec.tofile(tmp_path / f"data_batch_{i}.bin")
    c = V.CIFAR10(str(tmp_path), train=True)
    assert len(c) == 20 and c[0][0].shape == (3, 32, 32) and c[0][1] == 9 and c.as_tensors()[0].shape == (20, 3, 32, 32)
    rec100 = np.zeros((3, 3074), dtype=np.uint8)
    rec100[:, 1] = [42, 7, 99]
    rec100.tofile(tmp_path / "test.bin")
    assert V.CIFAR100(str(tmp_path), train=False)[2][1] == 99
    for cls in ("cat", "dog"):
        os.makedirs(tmp_path / "folder" / cls)
    np.save(tmp_path / "folder" / "cat" / "a.npy", (np.random.rand(6, 7, 3) * 255).astype(np.uint8))
    with open(tmp_path / "folder" / "dog" / "b.ppm", "wb") as f:
        f.write(b"P6\n# comment\n4 2\n255\n" + bytes(range(24)))
    fo = V.ImageFolder(str(tmp_path / "folder"))
    assert fo.classes == ["cat", "dog"] and fo[0][0].shape == (3, 6, 7) and fo[1][0].shape == (3, 2, 4) and fo[1][1] == 1
    with pytest.raises(FileNotFoundError):
        V.MNIST(str(tmp_path), train=False)


# ------------------------------------------------------------------ visualization
def test_training_plots_and_dashboard(tmp_path):
    pl = Z.TrainingPlotter()
    svg = pl.plot_training_curves({"train_loss": [3.0, 2.0, 1.5], "val_loss": [3.2, 2.4, 2.0]})
    assert svg.startswith("<svg") and svg.count("<polyline") == 2 and "validation" in svg
    cmp_ = pl.plot_loss_comparison({"a": [1, 0.5], "b": [1, 0.7], "c": [1, 0.9]})
    assert cmp_.count("<polyline") == 3
    dash = Z.create_dashboard([("curves", svg), ("cmp", cmp_)])
    Z.save_plot(dash, str(tmp_path / "d.html"))
    assert (tmp_path / "d.html").read_text().count("<svg") == 2
    Z.save_plot(svg, str(tmp_path / "p.html"), Z.PlotFormat.HTML)
    assert (tmp_path / "p.html").read_text().lower().startswith("<!doctype")
    assert 'width="100"' in Z.resize_svg(svg, 100, 50) and Z.generate_filename("x", Z.PlotFormat.SVG) == "x.svg"
    assert Z.PlotFormat.SVG.mime_type() == "image/svg+xml" and len(Z.ColorPalette.categorical()) == 10


def test_tensor_and_graph_visualizers():
    tv = Z.TensorVisualizer()
    hm = tv.heatmap(torch.randn(100, 300), "w")
    assert hm.count("<rect") == 64 * 64
    assert "<rect" in tv.histogram(torch.randn(1000), bins=10)
    st = tv.stats(torch.tensor([0.0, 1.0, 3.0]))
    assert st["max"] == 3 and st["sparsity"] == pytest.approx(1 / 3)
    x = torch.randn(2, 3, requires_grad=True)
    dot = Z.GraphVisualizer().autograd_dot((x * 2).sum())
    assert "MulBackward0" in dot and "SumBackward0" in dot and "->" in dot
    m = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.ReLU())
    md = Z.GraphVisualizer().module_dot(m)
    assert "Linear" in md and "15 params" in md
    assert Z.GraphVisualizer().module_svg(m).count("<rect") == 3


# ------------------------------------------------------------------ quantization
def test_quantize_dequantize_schemes():
    torch.manual_seed(0)
    x = torch.randn(64, 32) * 3
    for scheme in Q.QuantizationScheme:
        q = Q.quantize_tensor(x, Q.QuantizationConfig(scheme=scheme))
        err = (q.dequantize() - x).abs().max()
        assert err <= float(q.scale.max()) * 0.51 + 1e-6, scheme
    q4 = Q.quantize_tensor(x, Q.QuantizationConfig(qtype=Q.QuantizationType.INT4))
    assert q4.data.min() >= -8 and q4.data.max() <= 7
    packed = q4.pack_int4()
    assert packed.numel() == x.numel() // 2 and torch.equal(Q.QuantizedTensor.unpack_int4(packed, x.numel()).reshape(x.shape), q4.data)
    pc = Q.quantize_tensor(x, Q.QuantizationConfig(scheme=Q.QuantizationScheme.PER_CHANNEL_SYMMETRIC))
    assert pc.scale.shape == (64,) and Q.QuantizationType.INT4.range() == (-8, 7) and Q.QuantizationType.UINT8.bits() == 8
    with pytest.raises(ValueError):
        pc.reshape(32, 64)


def test_observers_and_static_quantizer():
    mm = Q.MinMaxObserver()
    mm.observe(torch.tensor([-1.0, 2.0]))
    mm.observe(torch.tensor([-3.0, 1.0]))
    lo, hi = mm.get_range()
    assert lo == -3 and hi == 2
    h = Q.HistogramObserver(bins=512)
    h.observe(torch.randn(10000))
    h.observe(torch.cat([torch.randn(10000), torch.tensor([40.0])]))      # outlier grows the range
    lo, hi = h.compute_optimal_range((0.001, 0.999))
    assert -5 < lo < -2 and 2 < hi < 5
    sq = Q.StaticQuantizer().with_calibration_method(Q.CalibrationMethod.MINMAX)
    Q.calibrate_batch(sq, [{"act": torch.randn(100)}, {"act": torch.randn(100) * 2}])
    assert sq.is_calibrated() and sq.get_params("act") is not None
    qt = sq.quantize("act", torch.randn(10))
    assert qt.data.dtype == torch.int8
    sq.reset()
    assert not sq.is_calibrated()
    for m in Q.CalibrationMethod:
        lo, hi = m.compute_range(torch.randn(5000))
        assert lo < 0 < hi


def test_quantized_ops_match_float():
    torch.manual_seed(1)
    a, b = torch.randn(24, 48), torch.randn(48, 16)
    qa = Q.quantize_tensor(a, Q.QuantizationConfig(scheme=Q.QuantizationScheme.ASYMMETRIC))
    qb = Q.quantize_tensor(b)
    acc, s = Q.QuantizedOps.qmatmul_int32(qa, qb)
    ref = qa.dequantize() @ qb.dequantize()
    assert torch.allclose(acc.float() * s, ref, atol=1e-3)
    assert (Q.QuantizedOps.qmatmul(qa, qb).dequantize() - a @ b).abs().max() < 0.6
    assert (Q.QuantizedOps.qadd(qa, qa).dequantize() - 2 * a).abs().max() < 0.1
    assert (Q.QuantizedOps.qmul(qa, qa).dequantize() - a * a).abs().max() < 0.2
    assert (Q.QuantizedOps.qrelu(qa).dequantize() - torch.relu(qa.dequantize())).abs().max() < 1e-6
    w = torch.randn(10, 48)
    qw = Q.quantize_tensor(w, Q.QuantizationConfig(scheme=Q.QuantizationScheme.PER_CHANNEL_SYMMETRIC))
    qx = Q.quantize_tensor(a)
    y = Q.qlinear(qx, qw, torch.ones(10))
    assert torch.allclose(y, qx.dequantize() @ qw.dequantize().t() + 1, atol=1e-3)


def test_qat_fake_quant_and_training():
    torch.manual_seed(2)
    fq = Q.FakeQuantize()
    x = torch.randn(100, requires_grad=True)
    y = fq(x)
    y.sum().backward()
    assert (y - x).abs().max() <= float(fq.scale) * 0.51 and x.grad.sum() == 100          # straight-through
    model = Q.prepare_qat(torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 1)))
    assert isinstance(model[0], Q.QATLinear)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    tr = Q.QATTrainer(Q.QATConfig(freeze_observer_after=5))
    X = torch.randn(64, 8)
    Y = X.sum(1, keepdim=True)
    losses = [tr.train_step(model, opt, torch.nn.functional.mse_loss, X, Y) for _ in range(40)]
    assert losses[-1] < losses[0] * 0.5 and not model[0].act_fq.observer_enabled
    tr.prepare_for_deployment(model)
    qw, bias = model[0].to_quantized()
    assert qw.data.dtype == torch.int8 and bias is not None
    conv = Q.QATConv2d(2, 3, 3, padding=1)
    assert conv(torch.randn(1, 2, 5, 5)).shape == (1, 3, 5, 5)


def test_qconv2d_integer_path_matches_dequantised_conv():
    import torch
    from rustorch_b200 import quantization as Q
    torch.manual_seed(0)
    img, filt = torch.randn(2, 3, 9, 9), torch.randn(5, 3, 3, 3) * 0.3
    qi = Q.quantize(img, torch.tensor(0.05), torch.tensor(2), Q.QuantizationType.INT8)
    qf = Q.quantize(filt, torch.tensor(0.01), torch.tensor(0), Q.QuantizationType.INT8)
    y = Q.QuantizedOps.qconv2d(qi, qf, torch.ones(5), stride=2, padding=1)
    ref = torch.nn.functional.conv2d(qi.dequantize(), qf.dequantize(), torch.ones(5), 2, 1)
    torch.testing.assert_close(y, ref, rtol=1e-4, atol=1e-4)
    acc = Q.int8_gemm(torch.tensor([[1, -2, 3]], dtype=torch.int8), torch.tensor([[4, 5, -6], [1, 1, 1]], dtype=torch.int8))
    assert acc.tolist() == [[-24, 2]]
