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
