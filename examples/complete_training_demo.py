"""A whole training job: data loaders, a trainer with gradient accumulation and clipping, metrics, checkpoints with a
retention policy, early stopping, then resuming from the best checkpoint (model and Adam moments) in a new process-like
state."""
import _path  # noqa: F401
import tempfile

import torch

from rustorch_b200 import data, nn, optim, training as T

torch.manual_seed(0)
X = torch.randn(512, 12)
y = (X[:, :4].sum(1) - X[:, 4:8].sum(1) > 0).long()
train = data.DataLoader(data.TensorDataset(X[:384], y[:384]), data.RandomSampler(384, seed=0), 32)
val = data.DataLoader(data.TensorDataset(X[384:], y[384:]), data.SequentialSampler(128), 64)


def make():
    m = nn.Sequential(nn.Linear(12, 32), nn.ReLU(), nn.Linear(32, 2))
    return m, optim.Adam(m.parameters(), lr=0.01)


model, opt = make()
ck = T.ModelCheckpoint(tempfile.mkdtemp(), monitor="val_loss", save_all=True, max_to_keep=3)
trainer = (T.TrainerBuilder().epochs(20).accumulation_steps(2).gradient_clip_value(1.0).metric("acc", T.accuracy)
           .callback(ck).callback(T.EarlyStopping("val_loss", patience=4)).build())
out = trainer.train(model, train, nn.CrossEntropyLoss(), opt, val_loader=val)
h = trainer.state.history
print(f"ran {out['epochs']} epochs, {out['steps']} optimizer steps; val loss {h[0].val_loss:.4f} -> {h[-1].val_loss:.4f}, accuracy {h[-1].metrics['acc']:.3f}")
print("checkpoints kept:", len(ck.manager.list()), " best epoch:", ck.manager.best().epoch)

m2, o2 = make()
extra = T.unpack_training_state(ck.manager.load_checkpoint(ck.manager.best()), m2, o2)
moments = sum(1 for s in o2.state_dict()["state"].values() if "exp_avg" in s)
ev = T.Trainer().evaluate(m2, val, nn.CrossEntropyLoss())
print(f"resumed from epoch {extra['epoch']}: {moments} parameter tensors with Adam moments, validation {({k: round(v, 4) for k, v in ev.items()})}")
