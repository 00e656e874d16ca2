"""The Python-binding surface of the reference resolves at the top level (and through the ``rustorch`` alias)."""
import pytest
import torch


def test_binding_surface_one_mlp_step():
    import rustorch as rt
    rt.set_seed(0)
    model = rt.Sequential(rt.Linear(4, 8), rt.ReLU(), rt.Linear(8, 1))
    opt = rt.SGD(model.parameters(), lr=0.1, momentum=0.9)
    x, y = torch.randn(32, 4), torch.randn(32, 1)
    loss_fn = rt.MSELoss()
    first = None
    for _ in range(30):
        opt.zero_grad()
        loss = loss_fn(model(x), y)
        loss.backward()
        opt.step()
        first = first if first is not None else float(loss)
    assert float(loss) < first
    t = rt.tensor([1.0, 2.0, 3.0, 4.0], [2, 2])
    assert list(t.shape()) == [2, 2]
    assert rt.zeros([2, 3]).numel() == 6 and rt.ones([2]).sum() is not None
    v = rt.Variable(rt.tensor([1.0, 2.0], [2]), requires_grad=True)
    (v * v).sum().backward()
    assert v.grad is not None
    with rt.no_grad():
        assert not torch.is_grad_enabled()


def test_helpers_device_config_comparator_transforms(tmp_path, monkeypatch):
    import rustorch_b200 as rt
    assert rt.Device("cuda:1").index == 1 and rt.Device.cpu().is_available() and not rt.Device.metal().is_available()
    with pytest.raises(ValueError):
        rt.Device("tpu")
    c = rt.Config(batch_size=32, use_amp="true")
    assert c.get_int("batch_size") == 32 and c.get_bool("use_amp")
    monkeypatch.setenv("RUSTORCH_BATCH_SIZE", "64")
    assert c.get_int("batch_size") == 64
    info = rt.get_system_info()
    assert "torch" in info and isinstance(rt.cuda_is_available(), bool)
    a, b = torch.nn.Linear(3, 2), torch.nn.Linear(3, 2)
    cmp_ = rt.ModelComparator.compare_parameters(a, b)
    assert not cmp_["identical"] and cmp_["max_abs_diff"] > 0
    b.load_state_dict(a.state_dict())
    assert rt.ModelComparator.compare_parameters(a, b)["identical"]
    assert rt.ModelComparator.compare_outputs(a, b, torch.randn(4, 3))["max_abs_diff"] == 0
    p = str(tmp_path / "m.rustorch")
    rt.ModelSerializer.save(a, p)
    c2 = torch.nn.Linear(3, 2)
    rt.ModelSerializer.load(c2, p)
    assert rt.ModelComparator.compare_parameters(a, c2)["identical"]
    tr = rt.Transforms.compose([rt.Transforms.resize(8), rt.Transforms.normalize([0.5], [0.5])])
    assert tr(torch.rand(1, 16, 16)).shape == (1, 8, 8)
    assert rt.DistributedConfig().backend == "nccl" and callable(rt.init_distributed) and rt.get_world_size() == 1 and rt.is_master()
    assert rt.functional.gelu(torch.zeros(2)).sum() == 0 and "Linear" in dir(rt)
    with pytest.raises(AttributeError):
        rt.does_not_exist


def test_layers_take_wrapper_tensors_and_variables():
    """The binding's layers map Variable to Variable (python/src/lib.rs:377-452): wrappers go through this package's
    layers, through plain torch.nn layers and through torch functions, and come back wrapped."""
    import rustorch as rt
    rt.set_seed(0)
    x = rt.tensor([[1.0, 2.0], [3.0, 4.0]])
    model = rt.Sequential(rt.Linear(2, 8), rt.ReLU(), rt.Linear(8, 1))
    opt = rt.Adam(model.parameters(), lr=1e-3)
    out = model(x)
    assert isinstance(out, rt.Tensor) and out.shape == [2, 1] and out.shape() == (2, 1)
    loss = rt.MSELoss()(out, rt.zeros([2, 1]))
    assert isinstance(loss, rt.Tensor) and float(loss) > 0 and f"{loss:.3f}" == f"{float(loss):.3f}"
    loss.backward()
    assert model[0].weight.grad is not None
    opt.step()
    opt.zero_grad()
    v = rt.Variable(x, requires_grad=True)
    o = model(v)
    assert isinstance(o, rt.Variable) and o.requires_grad and o.requires_grad()
    assert v.grad is None
    o.sum().backward()
    assert v.grad.shape == [2, 2] and v.grad().shape() == (2, 2) and v.data.numel == 4 and v.data().numel() == 4
    ref = model(x.data)                                               # plain torch tensor: plain torch result
    assert isinstance(ref, torch.Tensor) and torch.equal(ref, o.data.data)
    assert isinstance(torch.relu(x), rt.Tensor) and isinstance(torch.nn.functional.softmax(v, dim=-1), rt.Variable)
    assert isinstance(torch.cat([x, x]), rt.Tensor) and torch.cat([x, x]).shape == (4, 2)
    assert isinstance(torch.nn.Linear(2, 3)(x), rt.Tensor)            # a stock torch layer
    # a mixed call returns the Variable flavour; layers with several inputs and tuple outputs work too
    assert isinstance(rt.MSELoss()(o, rt.zeros([2, 1])), rt.Variable)
    seq, (h, c) = rt.LSTM(2, 3, batch_first=True)(rt.Variable(torch.randn(2, 5, 2)))
    assert isinstance(seq, rt.Variable) and isinstance(h, rt.Variable) and seq.shape == (2, 5, 3)
    att, w = rt.MultiheadAttention(4, 2)(rt.tensor(torch.randn(1, 3, 4)), rt.tensor(torch.randn(1, 3, 4)), rt.tensor(torch.randn(1, 3, 4)))
    assert isinstance(att, rt.Tensor) and att.shape == (1, 3, 4)
    img = rt.Conv2d(1, 2, (3, 3))(rt.Variable.randn([1, 1, 5, 5]))
    assert isinstance(img, rt.Variable) and img.shape == (1, 2, 3, 3)


def test_binding_accessors_attribute_and_call_spelling():
    """python/src/lib.rs declares shape / numel / ndim / data / grad / requires_grad / learning_rate ... as properties,
    src/python/*.rs as methods; both spellings work."""
    import copy
    import rustorch as rt
    t = rt.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [2, 3])
    assert t.shape == [2, 3] and t.shape == (2, 3) and t.shape() == (2, 3) and t.shape != [3, 2] and t.shape[1] == 3
    assert t.ndim == 2 and t.ndim() == 2 and t.numel == 6 and t.numel() == 6 and not t.requires_grad
    assert str(t.requires_grad) == "False" and len(t.shape) == 2 and {t.shape: 1}[(2, 3)] == 1
    v = rt.Variable.from_data([1.0, 2.0, 3.0, 4.0], [2, 2], True)
    assert v.requires_grad and v.numel == 4 and v.transpose().shape == (2, 2) and float(v.dot(v).item()) == 30.0
    assert rt.Variable.zeros([2, 3]).shape == (2, 3) and float(rt.Variable.ones([4]).sum().item()) == 4.0
    assert rt.Variable.randn([3, 3], requires_grad=True).requires_grad()
    assert not rt.Variable.ones([2], True).requires_grad_(False).requires_grad
    sh, dp = copy.copy(v), copy.deepcopy(v)
    assert sh.tensor is v.tensor and dp.tensor is not v.tensor and torch.equal(dp.tensor, v.tensor) and dp.requires_grad
    (v.exp().log() * v.sqrt().pow(2.0)).sum().backward()
    assert torch.allclose(v.grad.data, 2 * v.data.data)
    lin = rt.Linear(3, 2)
    sgd = rt.SGD(lin.parameters(), lr=0.1, momentum=0.9, nesterov=True, weight_decay=1e-4)
    assert sgd.learning_rate == pytest.approx(0.1) and sgd.learning_rate() == pytest.approx(0.1)
    assert sgd.momentum == pytest.approx(0.9) and sgd.nesterov and sgd.weight_decay() == pytest.approx(1e-4) and sgd.param_count() == 2
    with pytest.raises(AttributeError):
        sgd.beta1
    sgd.set_lr(0.05)
    assert sgd.learning_rate == pytest.approx(0.05)
    adam = rt.Adam(lin.parameters(), lr=1e-3, betas=(0.8, 0.9), eps=1e-6, amsgrad=True)
    assert (adam.beta1, adam.beta2, adam.eps) == (pytest.approx(0.8), pytest.approx(0.9), pytest.approx(1e-6)) and adam.amsgrad
    assert adam.step_count == 0
    lin(torch.randn(4, 3)).sum().backward()
    adam.step()
    adam.step()
    assert adam.step_count == 2 and adam.step_count() == 2
    from rustorch_b200.optim import StepLR
    sched = StepLR(adam, 1, 0.5)                                      # schedulers read the rate through either spelling
    sched.step()
    assert adam.learning_rate == pytest.approx(5e-4)


def test_binding_dataset_loader_sampler_backend():
    """src/python/data.rs and src/python/distributed.rs method sets."""
    import rustorch as rt
    xs, ys = torch.arange(20.0).view(10, 2), torch.arange(10.0).view(10, 1)
    ds = rt.TensorDataset(rt.tensor(xs), rt.tensor(ys))
    assert len(ds) == 10 and torch.equal(ds.data.data, xs) and torch.equal(ds.targets().data, ys)
    fx, fy = ds.get_batch([0, 9])
    assert torch.equal(fx, xs[[0, 9]]) and torch.equal(fy, ys[[0, 9]])
    with pytest.raises(IndexError):
        ds[10]
    assert len(rt.TensorDataset.from_tensors([xs, ys])) == 10
    dl = rt.DataLoader(ds, batch_size=4)
    assert dl.batch_size == 4 and dl.batch_size() == 4 and dl.num_batches() == 3 and len(dl) == 3 and dl.has_next()
    seen = []
    while dl.has_next():
        b = dl.next_batch()
        seen.append(b[0].shape[0])
    assert seen == [4, 4, 2] and dl.current_batch_index() == 3 and dl.next_batch() is None
    dl.reset()
    assert dl.current_batch_index() == 0 and dl.has_next() and [b[0].shape[0] for b in dl] == [4, 4, 2]
    with pytest.raises(ValueError):
        rt.DataLoader(ds, batch_size=0)
    # worker threads stay within the prefetch window, keep the order, hand errors to the consumer, stop when abandoned
    import threading
    import time

    class Slow(rt.Dataset):
        def __init__(self):
            self.loaded = 0

        def __len__(self):
            return 64

        def __getitem__(self, i):
            self.loaded += 1
            if i == 50:
                raise RuntimeError("bad sample")
            return torch.tensor([float(i)])

    slow = Slow()
    it = iter(rt.DataLoader(slow, batch_size=1, num_workers=2, prefetch=2))
    assert float(next(it)[0]) == 0.0
    time.sleep(0.2)
    assert slow.loaded <= 1 + 2 * 2 + 2                               # consumed + window + one in flight per worker
    got = [float(next(it)[0]) for _ in range(20)]
    assert got == [float(i) for i in range(1, 21)]
    with pytest.raises(RuntimeError, match="bad sample"):
        for _ in it:
            pass
    n_threads = threading.active_count()
    it2 = iter(rt.DataLoader(Slow(), batch_size=1, num_workers=2))
    next(it2)
    it2.close()                                                       # abandoned: the workers leave
    time.sleep(0.2)
    assert threading.active_count() <= n_threads
    from rustorch_b200.distributed import DistributedSampler
    s = DistributedSampler(10, 2, 1, seed=3)
    assert s.get_indices() == s.sample_indices() and len(s.get_indices()) == 5
    be = rt.DistributedBackend("gloo")
    assert be.backend_type == "gloo" and be.value == "gloo" and not be.is_initialized() and "gloo" in repr(be)
    one = rt.tensor([1.0, 2.0])
    assert be.all_reduce(one) is one and be.broadcast(one) is one and len(be.all_gather(one)) == 1      # no group: world of one
    be.barrier()
    with pytest.raises(ValueError):
        rt.DistributedBackend("carrier-pigeon")


def test_binding_model_builder_trainer_history():
    """src/python/training.rs: ModelBuilder.dense / conv2d / dropout / build, Model.add / compile / fit / evaluate /
    predict / summary on data loaders, Trainer(config).train / evaluate, TrainingHistory and TrainerConfig accessors.
    The reference's binding reports placeholder numbers there; these train."""
    import rustorch as rt
    rt.set_seed(0)
    X = torch.randn(256, 6)
    y = (X[:, :3].sum(1) > X[:, 3:].sum(1)).long()
    train = rt.DataLoader(rt.TensorDataset(X[:192], y[:192]), batch_size=32)
    val = rt.DataLoader(rt.TensorDataset(X[192:], y[192:]), batch_size=32)
    b = rt.ModelBuilder()
    b.dense(32, "relu")
    b.dropout(0.0)
    b.dense(2)
    assert repr(b) == "ModelBuilder(layers=3)"
    model = b.build("clf")
    assert isinstance(model, rt.Model) and "compiled=False" in repr(model)
    with pytest.raises(RuntimeError, match="compiled"):
        model.fit(train)
    with pytest.raises(RuntimeError, match="compiled"):
        model.evaluate(val)
    model.compile("adam", "cross_entropy", ["accuracy"], lr=0.02)
    hist = model.fit(train, val, epochs=12, verbose=False)
    assert isinstance(hist, rt.TrainingHistory) and len(hist.train_loss()) == 12 and len(hist.val_loss) == 12
    assert hist.train_loss[-1] < hist.train_loss[0] and hist.metrics()["accuracy"][-1] > 0.85
    assert hist.best_val_loss() == min(hist.val_loss()) and hist.val_loss[hist.best_epoch()] == hist.best_val_loss()
    assert hist.training_time > 0 and hist.training_time() >= sum(hist.epoch_time_s) * 0.5
    ep, tr, va = hist.plot_data()
    assert ep == [float(i) for i in range(1, 13)] and tr == hist.train_loss() and va == hist.val_loss()
    assert "12 epochs" in hist.summary() and "accuracy" in hist.summary()
    ev = model.evaluate(val)
    assert ev["accuracy"] > 0.85 and ev["loss"] == pytest.approx(hist.val_loss[-1], rel=1e-5)
    out = model.predict(rt.Variable(X[:5]))
    assert isinstance(out, rt.Variable) and out.shape == (5, 2)
    text = model.summary()
    assert "Model: clf" in text and "(Dense)" in text and "(None, 32)" in text and "Total params: 290" in text and "Compiled: True" in text
    # descriptions as strings, convolution with its input channels from the data, Dense flattening the feature map
    cnn = rt.Model("cnn")
    for spec in ("Conv2D(4, 3, activation=relu)", "Dropout(0.1)", "Dense(8, activation=tanh)", "Dense(3)"):
        cnn.add(spec)
    cnn.compile(None, None, None)                                     # binding defaults: sgd, mse, no extra metrics
    img = rt.DataLoader(rt.TensorDataset(torch.randn(16, 2, 6, 6), torch.randn(16, 3)), batch_size=8)
    h2 = cnn.fit(img, epochs=2, verbose=False)
    assert len(h2.train_loss) == 2 and h2.best_val_loss() is None and cnn.layers[0].inner.weight.shape == (4, 2, 3, 3)
    assert cnn.layers[2].inner.weight.shape == (8, 4 * 4 * 4) and cnn.predict(torch.randn(3, 2, 6, 6)).shape == (3, 3)
    with pytest.raises(ValueError):
        cnn.add("Banana(3)")
    with pytest.raises(ValueError):
        rt.ModelBuilder().dense(4, "nope")
    b2 = rt.ModelBuilder()
    b2.conv2d(4, 3, "relu")                                           # binding form
    b2.conv2d(4, 8, 3, 1, 1)                                          # explicit channels
    assert b2.build()(torch.randn(1, 2, 8, 8)).shape == (1, 8, 6, 6)
    # Trainer(config).train(model, loaders) -> history; evaluate -> metrics
    cfg = rt.TrainerConfig(epochs=3, learning_rate=0.01, batch_size=32, device="cpu")
    assert cfg.epochs == 3 and cfg.epochs() == 3 and cfg.device == "cpu" and cfg.device() == "cpu" and not cfg.use_mixed_precision()
    cfg.set_epochs(4)
    cfg.set_mixed_precision(False)
    cfg.set_device("cpu")
    cfg.log_frequency = 7
    assert cfg.epochs == 4 and cfg.log_frequency == 7 and "epochs=4" in repr(cfg) and cfg.learning_rate == pytest.approx(0.01)
    tr_ = rt.Trainer(cfg)
    h3 = tr_.train(model, train, val)
    assert isinstance(h3, rt.TrainingHistory) and len(h3.train_loss) == 4 and len(h3.val_loss) == 4
    m = tr_.evaluate(model, val)
    assert set(m) == {"loss", "accuracy"} and m["accuracy"] > 0.85 and "epochs=4" in repr(tr_)
    # stock torch loaders are accepted wherever this package's loaders are
    tl = torch.utils.data.DataLoader(torch.utils.data.TensorDataset(X[:64], y[:64]), batch_size=16)
    assert len(model.fit(tl, tl, epochs=2, verbose=False).val_loss) == 2 and "accuracy" in model.evaluate(tl)
    assert len(rt.Trainer(rt.TrainerConfig(epochs=1)).train(model, tl, tl).train_loss) == 1
    hh = rt.TrainingHistory()
    hh.add_epoch(0.5, 0.6, {"accuracy": 0.8})
    hh.add_epoch(0.4, 0.7)
    assert hh.train_loss() == [0.5, 0.4] and hh.val_loss() == [0.6, 0.7] and hh.best_epoch() == 0 and hh.metrics()["accuracy"] == [0.8]


def test_binding_utils_config_serializer_comparator_profiler(tmp_path):
    """src/python/utils.rs method sets."""
    import rustorch as rt
    c = rt.Config()
    assert c.get("device") == "cpu" and c.all()["num_threads"] == "4" and repr(c) == "Config(settings=5)"
    c.set("device", "cuda")
    c.set("lr", "0.01")
    path = str(tmp_path / "cfg.txt")
    c.save_to_file(path)
    c2 = rt.Config()
    c2.load_from_file(path)
    assert c2.get("device") == "cuda" and c2.get_float("lr") == 0.01 and c2.all() == c.all()
    c2.reset()
    assert c2.get("device") == "cpu" and c2.get("lr") is None
    with pytest.raises(FileNotFoundError):
        c2.load_from_file(str(tmp_path / "missing.txt"))
    b = rt.ModelBuilder()
    b.dense(4, "relu")
    b.dropout(0.1)
    b.dense(2)
    m1, m2 = b.build("a"), b.build("b")
    for m in (m1, m2):
        m.compile("sgd", "mse")
        m(torch.randn(1, 3))                                          # builds the described layers
    st = rt.ModelComparator.get_stats(m1)
    assert st["name"] == "a" and st["num_layers"] == 3 and st["dense_layers"] == 2 and st["dropout_layers"] == 1 and st["compiled"]
    assert st["parameters"] == 3 * 4 + 4 + 4 * 2 + 2
    cmp_ = rt.ModelComparator.compare(m1, m2)
    assert cmp_["layers_identical"] and cmp_["compilation_identical"] and cmp_["model2_name"] == "b"
    assert not cmp_["parameters_identical"]
    file = str(tmp_path / "m.safetensors")
    rt.ModelSerializer.export(m1, file, "safetensors")
    info = rt.ModelSerializer.get_model_info(file)
    assert info["exists"] and info["size"] > 0 and info["tensors"] == 4 and info["parameters"] == st["parameters"]
    assert rt.ModelSerializer.get_model_info(str(tmp_path / "none"))["exists"] is False
    assert len(rt.ModelSerializer.load(file)) == 4                    # path only: the tensors
    rt.ModelSerializer.load(m2, file)
    assert rt.ModelComparator.compare(m1, m2)["parameters_identical"]
    with pytest.raises(ValueError, match="Unsupported export format"):
        rt.ModelSerializer.export(m1, file, "docx")
    p = rt.Profiler()
    p.record("matmul", 1.0)                                           # disabled: ignored
    p.enable()
    for d in (0.5, 1.5, 1.0):
        p.record("matmul", d)
    with p.profile("scope"):
        pass
    s = p.get_stats()
    assert s["matmul"] == {"count": 3.0, "total": 3.0, "mean": 1.0, "min": 0.5, "max": 1.5} and s["scope"]["count"] == 1.0
    p.clear()
    assert p.get_stats() == {}


def test_binding_visualization(tmp_path):
    """src/python/visualization.rs: Plotter, ModelVisualizer, TensorStats draw (SVG / Graphviz text) instead of printing."""
    import rustorch as rt
    pl = rt.Plotter("svg", "default", (8, 4), 100)
    assert "figure_size=(8, 4)" in repr(pl) and pl.config.width == 640
    h = rt.TrainingHistory()
    for i in range(5):
        h.add_epoch(1.0 / (i + 1), 1.2 / (i + 1))
    out = str(tmp_path / "hist.svg")
    svg = pl.plot_training_history(h, out, True)
    assert svg.startswith("<svg") and svg.count("<polyline") == 2 and open(out).read() == svg
    assert pl.plot_training_history(h, None, False).count("<polyline") == 1
    assert pl.plot_tensor_as_image(rt.tensor(torch.randn(4, 6)), "w").count("<rect") == 24
    grid = pl.plot_multiple_tensors([torch.randn(2, 2), torch.randn(3, 3), torch.randn(2, 2)], ["a", "b", "c"], (2, 2))
    assert grid.count("<svg") == 3 and grid.count("<tr>") == 2
    with pytest.raises(ValueError):
        pl.plot_multiple_tensors([torch.randn(2, 2)] * 3, None, (1, 2))
    assert "<polyline" in pl.line_plot([0, 1, 2], [1.0, 4.0, 9.0], "squares", "n", "n^2") and "squares" in pl.line_plot([0, 1], [0, 1], "squares")
    with pytest.raises(ValueError):
        pl.line_plot([0, 1], [1.0])
    sc = pl.scatter_plot([0, 1, 2], [2, 1, 0], colors=[0.0, 0.5, 1.0], sizes=[2, 4, 6])
    assert sc.count("<circle") == 3 and 'r="6.0"' in sc
    with pytest.raises(ValueError):
        pl.scatter_plot([0, 1], [1, 2], sizes=[1])
    hs = pl.histogram(torch.randn(500).tolist(), 20, "h")
    assert hs.count('<rect x=') >= 15
    mv = rt.ModelVisualizer("dot", True, True)
    b = rt.ModelBuilder()
    b.dense(8, "relu")
    b.dense(2)
    model = b.build("viz")
    model.compile("sgd", "mse")
    model(torch.randn(1, 4))
    dot = mv.visualize_model(model.summary(), str(tmp_path / "m.dot"))
    assert dot.startswith("digraph model") and "l0 -> l1" in dot and "(None, 8)" in dot and open(tmp_path / "m.dot").read() == dot
    assert mv.visualize_model(model.summary(), None, "svg").count("<rect x=") == 2
    assert mv.visualize_model(model).startswith("digraph")
    att = torch.softmax(torch.randn(2, 3, 3), -1)                     # heads averaged
    hm = mv.plot_attention_heatmap(att, ["a", "b", "c"], "attn")
    assert hm.count("<rect x=") == 9 and hm.count(">a<") == 2
    with pytest.raises(ValueError):
        mv.plot_attention_heatmap(att, ["a", "b"])
    ts = rt.TensorStats(rt.tensor([4.0, 1.0, 3.0, 2.0]))
    with pytest.raises(RuntimeError):
        ts.get_stats()
    ts.compute_stats()
    st = ts.get_stats()
    assert st["count"] == 4 and st["mean"] == 2.5 and st["min"] == 1.0 and st["max"] == 4.0 and st["median"] == 3.0 and st["q25"] == 2.0
    assert st["q75"] == 4.0 and st["std"] == pytest.approx(1.118034, rel=1e-5) and ts.plot_stats(str(tmp_path / "s.svg")).startswith("<svg")
    with pytest.raises(ValueError):
        rt.TensorStats(torch.empty(0)).compute_stats()


def test_flows_of_the_reference_wheel_tests():
    """Call sequences of the reference's own Python tests (python/tests/test_phase3.py, test_phase4_*.py,
    test_phase5_autograd.py), re-expressed: optimizers over lists of Variables and of layer parameters, positional layer
    constructors, train / eval switches, ``rustorch.grad``."""
    import rustorch
    rustorch.set_seed(0)
    v = rustorch.Variable(rustorch.tensor([1.0, 2.0]), requires_grad=True)
    opt = rustorch.SGD([v], lr=0.1, momentum=0.0)
    (v * v).sum().backward()
    opt.step()
    assert v.data.as_slice() == pytest.approx([0.8, 1.6])            # the wrapped tensor was updated in place
    opt.zero_grad()
    assert v.grad is None
    adam = rustorch.Adam([v], lr=0.001, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, amsgrad=False)
    (v * 3.0).sum().backward()
    adam.step()
    assert v.data.as_slice() == pytest.approx([0.799, 1.599], abs=1e-5)
    X = rustorch.Variable(rustorch.tensor([1.0, 2.0]), requires_grad=False)
    y = rustorch.Variable(rustorch.tensor([1.0]), requires_grad=False)
    l1, l2 = rustorch.Linear(2, 4, True), rustorch.Linear(4, 1, True)
    relu, sig, crit = rustorch.ReLU(), rustorch.Sigmoid(), rustorch.MSELoss()
    sgd = rustorch.SGD([l1.weight, l1.bias, l2.weight, l2.bias], lr=0.5, momentum=0.0)
    losses = []
    for _ in range(20):
        sgd.zero_grad()
        loss = crit(sig(l2(relu(l1(X)))), y)
        loss.backward()
        sgd.step()
        losses.append(float(loss.item()))
    assert isinstance(loss, rustorch.Variable) and losses[-1] < losses[0]
    with pytest.raises(ValueError):
        rustorch.Linear(0, 5, True)
    assert rustorch.Linear(3, 2, bias=False).bias is None
    # CNN stack with positional constructor arguments, in training and evaluation mode
    layers = [rustorch.Conv2d(1, 4, (3, 3), (1, 1), (1, 1), True), rustorch.BatchNorm2d(4, 1e-5, 0.1, True), rustorch.ReLU(),
              rustorch.MaxPool2d((2, 2), (2, 2), (0, 0)), rustorch.Flatten(1, -1), rustorch.Linear(4 * 4 * 4, 8, True),
              rustorch.BatchNorm1d(8, 1e-5, 0.1, True, True), rustorch.Dropout(0.5, False), rustorch.Linear(8, 3, True)]
    params = [p for l in layers for p in (getattr(l, "weight", None), getattr(l, "bias", None)) if p is not None]
    opt2 = rustorch.Adam(params, lr=0.01, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, amsgrad=False)
    img = rustorch.Variable(rustorch.tensor(torch.randn(6, 1, 8, 8)), requires_grad=False)
    tgt = rustorch.Variable(rustorch.tensor(torch.tensor([0.0, 1.0, 2.0, 0.0, 1.0, 2.0])), requires_grad=False)
    ce = rustorch.CrossEntropyLoss()

    def run(x):
        for l in layers:
            x = l(x)
        return x

    first = None
    for _ in range(15):
        for l in layers:
            l.train()
        opt2.zero_grad()
        loss = ce(run(img), tgt)
        loss.backward()
        opt2.step()
        first = first if first is not None else float(loss.item())
    for l in layers:
        l.eval()
    out = run(img)
    assert isinstance(out, rustorch.Variable) and out.shape == (6, 3) and float(loss.item()) < first
    assert torch.equal(run(img).tensor, out.tensor)                   # evaluation mode: dropout off, running statistics
    a = rustorch.Variable(rustorch.tensor([2.0, 3.0]), requires_grad=True)
    yv = (a * a).sum()
    g = rustorch.grad([yv], [a], retain_graph=False, create_graph=False)
    assert g[0].as_slice() == [4.0, 6.0]
    with rustorch.no_grad():
        assert not (a * 2.0).requires_grad
    with rustorch.enable_grad():
        assert (a * 2.0).requires_grad


def test_alias_package_shares_modules_and_functional_namespace():
    """``import rustorch.nn`` must give the same module object as ``rustorch_b200.nn`` (one copy of every class), and
    ``rustorch.nn.functional`` has the stateless forms (python/python/rustorch/nn.py:444-464)."""
    import rustorch
    import rustorch.nn as N
    import rustorch.optim
    import rustorch_b200
    from rustorch.models.high_level import ModelBuilder
    from rustorch.nn import functional as F
    assert N is rustorch_b200.nn and F is rustorch_b200.nn.functional and rustorch.optim is rustorch_b200.optim
    assert ModelBuilder is rustorch_b200.models.high_level.ModelBuilder and rustorch.functional is F
    with pytest.raises(ImportError):
        import rustorch.does_not_exist  # noqa: F401
    assert rustorch.is_tensor(rustorch.tensor([1.0])) and not rustorch.is_tensor(torch.ones(1))
    v = rustorch.Variable(rustorch.tensor([[-1.0, 2.0]]), requires_grad=True)
    assert isinstance(N.Linear(2, 3)(v), rustorch.Variable)
    r = F.relu(v)
    assert isinstance(r, rustorch.Variable) and r.data.as_slice() == [0.0, 2.0]
    assert float(F.mse_loss(v, rustorch.Variable(rustorch.zeros([1, 2]))).item()) == 2.5
    ce = F.cross_entropy(v, rustorch.tensor([1.0]))                  # class index held in a float tensor
    assert isinstance(ce, rustorch.Variable) and float(ce.item()) == pytest.approx(0.048587, rel=1e-4)
    soft = F.cross_entropy(torch.tensor([[-1.0, 2.0]]), torch.tensor([[0.25, 0.75]]))      # a distribution stays one
    assert float(soft) == pytest.approx(0.25 * 3.048587 + 0.75 * 0.048587, rel=1e-4)
    assert float(N.CrossEntropyLoss()(torch.tensor([[-1.0, 2.0]]), torch.tensor([[0.25, 0.75]]))) == pytest.approx(float(soft))
    assert F.softmax(torch.zeros(2)).tolist() == [0.5, 0.5] and F.max_pool2d(torch.randn(1, 1, 4, 4), 2).shape == (1, 1, 2, 2)
    assert F.linear(v, torch.ones(3, 2)).shape == (1, 3) and F.one_hot(rustorch.tensor([1.0, 0.0]), 3).shape == (2, 3)
    assert F.layer_norm(torch.randn(2, 4), 4).shape == (2, 4) and F.silu(torch.zeros(1)).item() == 0.0


def test_described_layers_load_checkpoints_before_seeing_data(tmp_path):
    """A freshly built Keras-like model (layers not materialised yet) loads a saved one in every file format, and a
    strict load does not drop names it does not know."""
    import rustorch as rt
    b = rt.ModelBuilder()
    b.conv2d(4, 3, "relu")
    b.dense(8, "relu")
    b.dense(2)
    src = b.build("src")
    x = torch.randn(2, 3, 6, 6)
    want = src(x)
    for fmt, name in (("safetensors", "m.safetensors"), ("rustorch", "m.rustorch"), ("pytorch", "m.pt")):
        path = str(tmp_path / name)
        rt.ModelSerializer.export(src, path, fmt)
        fresh = b.build("fresh")
        assert fresh.layers[0].inner is None
        rt.ModelSerializer.load(fresh, path)
        assert torch.equal(fresh(x), want), fmt
    third = b.build("third")
    third.load_state_dict(src.state_dict())
    assert torch.equal(third(x), want)
    other = rt.ModelBuilder()
    other.dense(9)
    with pytest.raises(ValueError, match="8 units"):
        other.build().load_state_dict({"layers.0.inner.weight": torch.zeros(8, 4), "layers.0.inner.bias": torch.zeros(8)})
    plain = torch.nn.Linear(4, 2)
    extra = str(tmp_path / "extra.safetensors")
    from rustorch_b200.formats import save_safetensors
    save_safetensors({"weight": torch.zeros(2, 4), "bias": torch.zeros(2), "ghost": torch.zeros(1)}, extra)
    with pytest.raises(RuntimeError, match="ghost"):
        rt.ModelSerializer.load(plain, extra)                        # strict: the unknown name is reported
    rt.ModelSerializer.load(plain, extra, strict=False)
    assert float(plain.weight.abs().sum()) == 0.0


def test_callback_registry_result_and_try_catch():
    """The binding's host-callback utilities (python/tests/test_advanced.py:9-150, test_direct.py:16-30), reachable
    through the extension module's own name too."""
    import rustorch as rt
    import _rustorch_py as ext
    assert ext is rt
    reg = rt.init_callback_system()
    reg.register_callback("my_callback", lambda m: f"Python received: {m}")
    reg.register_callback("progress", lambda s, t, p: f"Progress: {s}/{t} ({p:.1f}%)")
    reg.register_callback("completed", lambda n: f"Completed {n} operations")
    assert reg.list_callbacks() == ["completed", "my_callback", "progress"] and "progress" in reg and len(reg) == 3
    assert rt.call_python_from_rust(reg, "my_callback", "hi") == "Python received: hi"
    assert rt.progress_callback_example(reg, 4) == ["Progress: 1/4 (25.0%)", "Progress: 2/4 (50.0%)", "Progress: 3/4 (75.0%)",
                                                    "Progress: 4/4 (100.0%)", "Completed 4 operations"]
    with pytest.raises(rt.RusTorchError, match="no callback named 'nope'"):
        reg.call("nope")
    with pytest.raises(rt.RusTorchError):
        reg.register_callback("x", 3)
    assert reg.unregister_callback("completed") and not reg.unregister_callback("completed")
    e = rt.RusTorchError("Test error", 1001)
    assert e.message == "Test error" and e.error_code == 1001 and "Test error" in str(e)
    ok, err = rt.Result.ok("v"), rt.Result.err("bad")
    assert ok.is_ok and not ok.is_err and err.is_err and ok.unwrap() == "v" and err.unwrap_or("d") == "d" and ok.unwrap_or("d") == "v"
    with pytest.raises(rt.RusTorchError, match="bad"):
        err.unwrap()
    with pytest.raises(KeyError):
        rt.Result.err(KeyError("k")).unwrap()
    assert ok.map(str.upper).unwrap() == "V" and err.map(str.upper) is err and err.unwrap_err() == "bad" and repr(ok) == "Ok('v')"
    assert rt.try_catch(lambda: "Success!") == "Success!"
    assert rt.try_catch(lambda: 1 / 0, lambda ex: f"handled {type(ex).__name__}") == "handled ZeroDivisionError"
    with pytest.raises(ZeroDivisionError):
        rt.try_catch(lambda: 1 / 0)
    assert rt.get_version() == rt.__version__ and "RusTorch" in rt.hello_from_rust()
    assert rt.add_numbers(1.5, 2.5) == 4.0 and rt.sum_list([1.0, 2.0, 3.0, 4.0, 5.0]) == 15.0


def test_trainer_reports_through_a_callback_registry():
    import rustorch as rt
    from rustorch_b200.training import Trainer, TrainerConfig
    torch.manual_seed(0)
    seen, logs = [], []
    reg = rt.init_callback_system()
    reg.register_callback("progress", lambda s, t, p: seen.append((s, t, round(p))) or (s < 3))      # False at epoch 3: stop
    reg.register_callback("log", lambda level, text: logs.append((level, text)))
    reg.register_callback("completed", lambda n: seen.append(("done", n)))
    model = torch.nn.Linear(4, 1)
    data = [(torch.randn(8, 4), torch.randn(8, 1)) for _ in range(3)]
    cfg = TrainerConfig()
    cfg.epochs = 5
    Trainer(cfg, callbacks=reg).train(model, data, torch.nn.MSELoss(), torch.optim.SGD(model.parameters(), lr=0.01))
    assert seen == [(1, 5, 20), (2, 5, 40), (3, 5, 60), ("done", 3)]
    assert len(logs) == 3 and logs[0][0] == "info" and logs[0][1].startswith("epoch 1/5: train_loss ")
