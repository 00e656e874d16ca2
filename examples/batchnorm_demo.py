"""BatchNorm in training and evaluation mode, running statistics, and the other normalisation layers side by side."""
import _path  # noqa: F401

import torch

from rustorch_b200 import nn

torch.manual_seed(0)
x = torch.randn(64, 8) * 3 + 5
bn = nn.BatchNorm1d(8)
y = bn(x)
print("train mode: output mean %.4f var %.4f" % (float(y.detach().mean()), float(y.detach().var(unbiased=False))))
print("running mean moved by momentum 0.1: %.3f (batch mean %.3f)" % (float(bn.running_mean.mean()), float(x.mean())))
bn.eval()
print("eval mode uses the running statistics: mean of output %.3f, is_training %s" % (float(bn(x).detach().mean()), bn.is_training()))
img = torch.randn(4, 6, 5, 5) * 2 + 1
for name, layer in (("BatchNorm2d", nn.BatchNorm2d(6)), ("GroupNorm(3 groups)", nn.GroupNorm(3, 6)), ("InstanceNorm2d", nn.InstanceNorm2d(6)),
                    ("LayerNorm([6, 5, 5])", nn.LayerNorm([6, 5, 5]))):
    out = layer(img)
    print(f"{name:<22} per-sample mean {float(out[0].mean()):+.4f}  per-channel mean {float(out[:, 0].mean()):+.4f}")
r = nn.RMSNorm(8)
print("RMSNorm: root mean square of each row = %.4f" % float(r(x).pow(2).mean(-1).sqrt().mean()))
