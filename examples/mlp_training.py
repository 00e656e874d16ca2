"""MLP 784 -> 256 -> 128 -> 10 trained with Adam on synthetic data through DataLoader and Trainer."""
import _path  # noqa: F401
import tempfile

import torch

from rustorch_b200 import data, nn, optim, training

dev = "cuda" if torch.cuda.is_available() else "cpu"
torch.manual_seed(0)
xs, ys = torch.randn(2048, 784), torch.randint(0, 10, (2048,))
loader = data.DataLoader(data.TensorDataset(xs, ys), batch_size=128, shuffle=True)
model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 10)).to(dev)
opt = optim.Adam(model.parameters(), lr=1e-3)
loss_fn = nn.CrossEntropyLoss()

for epoch in range(3):
    total = 0.0
    for xb, yb in loader:
        xb, yb = xb.to(dev), yb.to(dev)
        opt.zero_grad()
        loss = loss_fn(model(xb), yb)
        loss.backward()
        opt.step()
        total += float(loss)
    print(f"epoch {epoch}: mean loss {total / len(loader):.4f}")

with tempfile.TemporaryDirectory() as d:
    mgr = training.CheckpointManager(training.SaveConfig(directory=d, monitor="loss"))
    meta = mgr.save_checkpoint(3, 3 * len(loader), {"loss": total / len(loader)}, training.pack_training_state(model, opt))
    print("checkpoint:", meta.name, "best loss so far:", mgr.best_value())
