"""Trainer / callbacks / checkpoint manager / AMP / data loaders on CPU, incl. the MLP config:
784 -> 256 -> 128 -> 10 with ReLU, batch 64, N(0,1) inputs, uniform labels, cross-entropy, Adam lr 1e-3, seed 0."""
import math
import os

import pytest
import torch

from rustorch_b200 import amp, data, nn, optim, training as T


def _toy(n=64):
    g = torch.Generator().manual_seed(0)
    X = torch.randn(n, 8, generator=g)
    y = (X[:, 0] > 0).long()
    return data.TensorDataset(X, y)


def test_dataset_samplers_loader():
    ds = _toy(10)
    assert len(ds) == 10 and ds[3][0].shape == (8,)
    cat = data.ConcatDataset([ds, ds])
    assert len(cat) == 20 and torch.equal(cat[13][0], ds[3][0])
    assert list(data.SequentialSampler(4)) == [0, 1, 2, 3]
    a, b = list(data.RandomSampler.with_seed(10, 5)), list(data.RandomSampler.with_seed(10, 5))
    assert sorted(a) == list(range(10)) and a == b
    assert len(list(data.RandomSampler.with_replacement(3, 9))) == 9
    assert sorted(data.SubsetRandomSampler([2, 5, 7])) == [2, 5, 7]
    w = list(data.WeightedRandomSampler([0.0, 1.0, 0.0], 20, seed=0))
    assert set(w) == {1}
    assert [len(x) for x in data.BatchSampler(data.SequentialSampler(10), 4)] == [4, 4, 2]
    dl = data.DataLoader(ds, data.SequentialSampler(10), 4)
    assert len(dl) == 3 and dl.next_batch()[0].shape == (4, 8)
    dl.reset()
    n = 0
    while dl.next_batch() is not None:
        n += 1
    assert n == 3
    threaded = data.DataLoader.with_options(ds, data.SequentialSampler(10), 3, num_workers=2)
    seq = torch.cat([b[0] for b in threaded])
    assert torch.equal(seq, ds.tensors[0])          # worker threads keep batch order


def test_trainer_steps_and_callbacks(tmp_path):
    torch.manual_seed(0)
    ds = _toy(64)
    model = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 2))
    opt = optim.Adam(model.parameters(), lr=0.05)
    ck = T.ModelCheckpoint(str(tmp_path / "ck"), monitor="val_loss", save_all=True, max_to_keep=2)
    prog = T.ProgressBar(log_frequency=2)
    tr = (T.TrainerBuilder().epochs(6).accumulation_steps(2).gradient_clip_value(1.0).validation_frequency(1)
          .metric("acc", T.accuracy).callback(ck).callback(prog).callback(T.EarlyStopping("val_loss", patience=50)).build())
    loader = data.DataLoader(ds, data.SequentialSampler(64), 16)
    w0 = model[0].weight.detach().clone()
    out = tr.train(model, loader, nn.CrossEntropyLoss(), opt, val_loader=loader)
    assert not torch.equal(model[0].weight, w0)                       # the optimizer really stepped
    assert out["steps"] == 6 * 2                                       # 4 batches / accumulation 2
    h = tr.state.history
    assert h[-1].train_loss < h[0].train_loss and h[-1].metrics["acc"] > 0.8 and h[-1].val_loss is not None
    assert len(ck.manager.list()) == 2 and ck.manager.best() is not None
    assert any("done" in l for l in prog.lines)
    # resume: state (incl. Adam moments) comes back
    m2 = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 2))
    o2 = optim.Adam(m2.parameters(), lr=0.05)
    extra = T.unpack_training_state(ck.manager.load_checkpoint(), m2, o2)
    assert torch.equal(m2[0].weight, model[0].weight) and extra["epoch"] == 5
    assert any("exp_avg" in s for s in o2.state_dict()["state"].values())


def test_early_stopping_and_checkpoint_policy(tmp_path):
    es = T.EarlyStopping("val_loss", patience=2)
    st = T.TrainingState()
    sig = [es.on_epoch_end(st, T.EpochState(i, 1.0, v)) for i, v in enumerate([1.0, 0.9, 0.95, 0.97])]
    assert sig[-1] is T.CallbackSignal.STOP and sig[:3] == [None, None, None]
    cm = T.CheckpointManager(T.SaveConfig(str(tmp_path / "c"), max_to_keep=2, monitor="loss"))
    for i, l in enumerate([0.5, 0.3, 0.4, 0.45]):
        cm.save_checkpoint(i, i * 10, {"loss": l}, b"x" * (i + 1))
    names = [c.epoch for c in cm.list()]
    assert 1 in names and len(names) == 2 and cm.best().epoch == 1 and cm.latest().epoch == 3
    assert cm.load_checkpoint(cm.best()) == b"xx"
    assert T.CheckpointManager(T.SaveConfig(str(tmp_path / "c"), monitor="loss")).best().epoch == 1   # index reload
    bo = T.CheckpointManager(T.SaveConfig(str(tmp_path / "b"), monitor="loss", save_best_only=True))
    assert bo.save_checkpoint(0, 0, {"loss": 1.0}, b"a") is not None and bo.save_checkpoint(1, 1, {"loss": 2.0}, b"b") is None
    cmx = T.ConfusionMatrix(2)
    cmx.update(torch.tensor([0, 1, 1, 1]), torch.tensor([0, 1, 0, 1]))
    assert cmx.accuracy() == 0.75 and cmx.recall().tolist() == [0.5, 1.0]


def test_grad_scaler_and_amp_optimizer():
    s = amp.GradScaler()
    assert (s.get_scale(), s.growth_factor, s.backoff_factor, s.growth_interval) == (65536.0, 2.0, 0.5, 2000)
    p = torch.nn.Parameter(torch.ones(2))
    o = torch.optim.SGD([p], lr=1.0)
    s.scale((p * 2).sum()).backward()
    assert p.grad.tolist() == [131072.0, 131072.0]
    assert s.step(o) and p.tolist() == [-1.0, -1.0]                 # unscaled gradient 2
    s.update_scale()
    p.grad = torch.tensor([float("inf"), 1.0])
    assert not s.step(o) and p.tolist() == [-1.0, -1.0]             # overflow: step skipped
    s.update_scale()
    assert s.get_scale() == 32768.0 and s.overflow_count == 1
    g = amp.GradScaler(init_scale=4.0, growth_interval=2)
    for _ in range(2):
        p.grad = torch.ones(2)
        g.step(o)
        g.update_scale()
    assert g.get_scale() == 8.0
    sd = g.state_dict()
    g2 = amp.GradScaler()
    g2.load_state_dict(sd)
    assert g2.get_scale() == 8.0
    ao = amp.AMPOptimizer(torch.optim.SGD([p], lr=0.1), amp.AMPConfig.fp16_static(8.0))
    with ao.autocast("cpu"):
        loss = (p * p).sum()
    ao.backward(loss)
    assert ao.step() and ao.success_rate() == 1.0
    with amp.autocast("cpu", dtype="bf16"):
        assert (torch.ones(2, 2) @ torch.ones(2, 2)).dtype == torch.bfloat16
    assert amp.AMPConfig.bf16().use_grad_scaler is False


def test_mlp_config_784_256_128_10_adam_100_steps():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(784, 256), torch.nn.ReLU(), torch.nn.Linear(256, 128), torch.nn.ReLU(),
                                torch.nn.Linear(128, 10))            # Kaiming-uniform init (torch default)
    assert sum(p.numel() for p in model.parameters()) == 235146
    opt = optim.Adam(model.parameters(), lr=1e-3)
    g = torch.Generator().manual_seed(0)
    X, y = torch.randn(64, 784, generator=g), torch.randint(0, 10, (64,), generator=g)
    ds = data.TensorDataset(X, y)
    tr = T.Trainer(T.TrainerConfig(epochs=100, log_frequency=0))
    out = tr.train(model, data.DataLoader(ds, data.SequentialSampler(64), 64), nn.CrossEntropyLoss(), opt)
    h = tr.state.history
    assert out["steps"] == 100 and abs(h[0].train_loss - math.log(10)) < 0.3 and h[-1].train_loss < 0.05
