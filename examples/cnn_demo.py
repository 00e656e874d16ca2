"""Small CNN on synthetic 32x32 images: Conv2d / BatchNorm2d / MaxPool2d, SGD with momentum."""
import _path  # noqa: F401
import torch

from rustorch_b200 import nn, optim

dev = "cuda" if torch.cuda.is_available() else "cpu"
dtype = torch.bfloat16 if dev == "cuda" else torch.float32
torch.manual_seed(0)
model = nn.Sequential(
    nn.Conv2d(3, 64, 3, padding=1), nn.BatchNorm2d(64), nn.ReLU(), nn.MaxPool2d(2),
    nn.Conv2d(64, 64, 3, padding=1), nn.BatchNorm2d(64), nn.ReLU(), nn.MaxPool2d(2),      # 64 -> 64, 3x3: resident-halo kernel on B200
    nn.Conv2d(64, 128, 3, stride=2, padding=1), nn.BatchNorm2d(128), nn.ReLU(),
    nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(128, 10),
).to(dev).to(memory_format=torch.channels_last).to(dtype)
opt = optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
x = torch.randn(64, 3, 32, 32, device=dev).to(dtype).contiguous(memory_format=torch.channels_last)
y = torch.randint(0, 10, (64,), device=dev)
for step in range(10):
    opt.zero_grad()
    loss = torch.nn.functional.cross_entropy(model(x).float(), y)
    loss.backward()
    opt.step()
    print(f"step {step}: loss {float(loss):.4f}")
