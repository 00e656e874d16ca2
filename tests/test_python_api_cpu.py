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
