"""Automatic mixed precision: ``autocast`` regions and a ``GradScaler`` that skips steps with inf / nan gradients."""
import _path  # noqa: F401
import torch

from rustorch_b200 import amp, nn, optim

dev = "cuda" if torch.cuda.is_available() else "cpu"
torch.manual_seed(0)
model = nn.Sequential(nn.Linear(64, 128), nn.GELU(), nn.Linear(128, 8)).to(dev)
opt = optim.SGD(model.parameters(), lr=0.05)
scaler = amp.GradScaler()
x, y = torch.randn(256, 64, device=dev), torch.randn(256, 8, device=dev)
for step in range(5):
    opt.zero_grad()
    with amp.autocast(device_type=dev):
        loss = torch.nn.functional.mse_loss(model(x).float(), y)
    scaler.scale(loss).backward()
    scaler.step(opt)
    scaler.update()
    print(f"step {step}: loss {float(loss):.4f} scale {scaler.get_scale():.0f}")
