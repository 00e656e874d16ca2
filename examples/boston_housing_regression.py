"""Tabular regression with an MLP, feature standardisation, a validation split and early stopping (the reference's
housing-price example; the table here is synthetic with the same 13-feature layout)."""
import _path  # noqa: F401

import torch

import rustorch as rt
from rustorch_b200.training import EarlyStopping, Trainer, TrainerConfig

rt.set_seed(1)
n, d = 506, 13
X = torch.randn(n, d) * torch.linspace(0.5, 3.0, d) + torch.linspace(-2, 2, d)
price = 22.0 + X[:, 5] * 3.0 - X[:, 12] * 2.0 + 0.5 * X[:, 0] * X[:, 5] + torch.randn(n)
mean, std = X[:400].mean(0), X[:400].std(0)
Xs = (X - mean) / std
train = rt.DataLoader(rt.TensorDataset(Xs[:400], price[:400].unsqueeze(1)), batch_size=32, shuffle=True)
val = rt.DataLoader(rt.TensorDataset(Xs[400:], price[400:].unsqueeze(1)), batch_size=64)
model = rt.Sequential(rt.Linear(d, 32), rt.ReLU(), rt.Linear(32, 16), rt.ReLU(), rt.Linear(16, 1))
trainer = Trainer(TrainerConfig(epochs=60, log_frequency=0), callbacks=[EarlyStopping("val_loss", patience=8)])
res = trainer.train(model, train, rt.MSELoss(), rt.Adam(model.parameters(), lr=5e-3), val)
pred = model(Xs[400:]).squeeze(1).detach()
rmse = float(((pred - price[400:]) ** 2).mean().sqrt())
base = float(((price[:400].mean() - price[400:]) ** 2).mean().sqrt())
print(f"epochs run: {res['epochs']}  validation RMSE {rmse:.3f}  (predicting the mean: {base:.3f})")
