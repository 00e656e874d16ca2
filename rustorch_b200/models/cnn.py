"""Convolutional models: ``CNN``, ``ResNet`` (18 / 34 with basic blocks, 50 with bottlenecks) and builders
(src/models/cnn.rs:17-776).

Same topology as the reference (7x7/2 stem + BN + ReLU + 3x3/2 max-pool, stages 64/128/256/512, 1x1
down-sampling shortcuts, ``fc 512 -> classes``) with its two omissions fixed: the residual addition is
really performed (commented out in cnn.rs:435-437) and the global average pool exists (empty in cnn.rs:551).
Built from the framework's ``Conv2d`` / ``BatchNorm2d``: in bf16 on CUDA (channels-last) the body convolutions run on
the implicit-GEMM tcgen05 kernels and every BatchNorm (+ residual add + ReLU) is one native kernel; the 3-channel
stem convolution, pooling and anything on CPU / fp32 use the library.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn.layers import AdaptiveAvgPool2d, BatchNorm2d, Conv2d, Dropout, MaxPool2d


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, in_ch: int, out_ch: int, stride: int = 1):
        super().__init__()
        self.conv1 = Conv2d(in_ch, out_ch, 3, stride, 1, bias=False)
        self.bn1 = BatchNorm2d(out_ch)
        self.conv2 = Conv2d(out_ch, out_ch, 3, 1, 1, bias=False)
        self.bn2 = BatchNorm2d(out_ch)
        self.downsample = None
        if stride != 1 or in_ch != out_ch:
            self.downsample = nn.Sequential(Conv2d(in_ch, out_ch, 1, stride, 0, bias=False), BatchNorm2d(out_ch))

    def forward(self, x):
        identity = x if self.downsample is None else self.downsample(x)
        out = self.bn1(self.conv1(x), relu=True)                       # BatchNorm + ReLU in one kernel
        return self.bn2(self.conv2(out), residual=identity, relu=True)  # BatchNorm + residual add + ReLU in one kernel


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, in_ch: int, mid: int, stride: int = 1):
        super().__init__()
        out_ch = mid * 4
        self.conv1 = Conv2d(in_ch, mid, 1, 1, 0, bias=False)
        self.bn1 = BatchNorm2d(mid)
        self.conv2 = Conv2d(mid, mid, 3, stride, 1, bias=False)
        self.bn2 = BatchNorm2d(mid)
        self.conv3 = Conv2d(mid, out_ch, 1, 1, 0, bias=False)
        self.bn3 = BatchNorm2d(out_ch)
        self.downsample = None
        if stride != 1 or in_ch != out_ch:
            self.downsample = nn.Sequential(Conv2d(in_ch, out_ch, 1, stride, 0, bias=False), BatchNorm2d(out_ch))

    def forward(self, x):
        identity = x if self.downsample is None else self.downsample(x)
        out = self.bn1(self.conv1(x), relu=True)
        out = self.bn2(self.conv2(out), relu=True)
        return self.bn3(self.conv3(out), residual=identity, relu=True)


class ResNet(nn.Module):
    def __init__(self, block, layers: Sequence[int], num_classes: int = 1000, in_channels: int = 3):
        super().__init__()
        self.in_ch = 64
        self.conv1 = Conv2d(in_channels, 64, 7, 2, 3, bias=False)
        self.bn1 = BatchNorm2d(64)
        self.maxpool = MaxPool2d(3, 2, 1)
        self.layer1 = self._make(block, 64, layers[0], 1)
        self.layer2 = self._make(block, 128, layers[1], 2)
        self.layer3 = self._make(block, 256, layers[2], 2)
        self.layer4 = self._make(block, 512, layers[3], 2)
        self.avgpool = AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(512 * block.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def _make(self, block, ch: int, n: int, stride: int) -> nn.Sequential:
        blocks = [block(self.in_ch, ch, stride)]
        self.in_ch = ch * block.expansion
        blocks += [block(self.in_ch, ch) for _ in range(1, n)]
        return nn.Sequential(*blocks)

    def forward(self, x):
        x = self.maxpool(self.bn1(self.conv1(x), relu=True))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(torch.flatten(self.avgpool(x), 1))

    @classmethod
    def from_torchvision(cls, source, **kw) -> "ResNet":
        """A model with the weights of a ``torchvision`` ResNet-18 / 34 / 50: ``source`` is that model, its ``state_dict()``
        or the path of a saved one (``.pth``).  Parameter and buffer names are torchvision's, so the tensors load as they
        are (stride on the 3x3 convolution of the bottleneck, as in torchvision); depth and class count are read from the
        tensors."""
        sd = source.state_dict() if isinstance(source, nn.Module) else source
        if isinstance(sd, (str, bytes)) or hasattr(sd, "__fspath__"):
            sd = torch.load(sd, map_location="cpu", weights_only=True)
        sd = sd.get("state_dict", sd) if isinstance(sd, dict) else sd
        sd = {k[7:] if k.startswith("module.") else k: v for k, v in sd.items()}
        try:
            depth = [1 + max(int(k.split(".")[1]) for k in sd if k.startswith(f"layer{i}.")) for i in (1, 2, 3, 4)]
            classes, width = sd["fc.weight"].shape
            in_ch = sd["conv1.weight"].shape[1]
        except (KeyError, ValueError):
            raise ValueError("not a torchvision ResNet state dict (conv1 / layer1..4 / fc expected)") from None
        bottleneck = any(k.endswith(".conv3.weight") for k in sd)
        c1, c2 = sd["layer1.0.conv1.weight"].shape, sd["layer1.0.conv2.weight"].shape
        if width != 512 * (4 if bottleneck else 1) or sd["conv1.weight"].shape[0] != 64 or c1[0] != 64 or c2[0] != c2[1]:
            raise ValueError(f"stage-1 convolutions {tuple(c1)} / {tuple(c2)}, fc input width {width}: wide and grouped variants are outside this model")
        model = cls(Bottleneck if bottleneck else BasicBlock, depth, int(classes), in_channels=int(in_ch), **kw)
        model.load_state_dict(sd, strict=True)
        return model

    @staticmethod
    def resnet18(num_classes: int = 1000, **kw) -> "ResNet":
        return ResNet(BasicBlock, [2, 2, 2, 2], num_classes, **kw)

    @staticmethod
    def resnet34(num_classes: int = 1000, **kw) -> "ResNet":
        return ResNet(BasicBlock, [3, 4, 6, 3], num_classes, **kw)

    @staticmethod
    def resnet50(num_classes: int = 1000, **kw) -> "ResNet":
        return ResNet(Bottleneck, [3, 4, 6, 3], num_classes, **kw)


resnet18, resnet34, resnet50 = ResNet.resnet18, ResNet.resnet34, ResNet.resnet50


class CNN(nn.Module):
    """Configurable conv stack + MLP classifier: ``CNN(input_shape (C,H,W), conv_channels, fc_sizes, num_classes)``."""

    def __init__(self, input_shape: Tuple[int, int, int] = (1, 28, 28), conv_channels: Sequence[int] = (32, 64),
                 fc_sizes: Sequence[int] = (128,), num_classes: int = 10, kernel_size: int = 3, dropout: float = 0.0,
                 batch_norm: bool = False):
        super().__init__()
        c, h, w = input_shape
        layers: List[nn.Module] = []
        for oc in conv_channels:
            layers.append(nn.Conv2d(c, oc, kernel_size, padding=kernel_size // 2))
            if batch_norm:
                layers.append(nn.BatchNorm2d(oc))
            layers += [nn.ReLU(), MaxPool2d(2)]
            c, h, w = oc, h // 2, w // 2
        self.features = nn.Sequential(*layers)
        fcs: List[nn.Module] = []
        d = c * h * w
        for s in fc_sizes:
            fcs += [nn.Linear(d, s), nn.ReLU()]
            if dropout:
                fcs.append(Dropout(dropout))
            d = s
        fcs.append(nn.Linear(d, num_classes))
        self.classifier = nn.Sequential(*fcs)

    def forward(self, x):
        return self.classifier(torch.flatten(self.features(x), 1))


class CNNBuilder:
    def __init__(self):
        self._kw = {}

    def input_shape(self, c, h, w):
        self._kw["input_shape"] = (c, h, w)
        return self

    def conv_channels(self, ch):
        self._kw["conv_channels"] = tuple(ch)
        return self

    def fc_sizes(self, s):
        self._kw["fc_sizes"] = tuple(s)
        return self

    def num_classes(self, n):
        self._kw["num_classes"] = n
        return self

    def dropout(self, p):
        self._kw["dropout"] = p
        return self

    def batch_norm(self, on=True):
        self._kw["batch_norm"] = on
        return self

    def build(self) -> CNN:
        return CNN(**self._kw)


class ResNetBuilder:
    def __init__(self):
        self._depth, self._classes, self._in = 18, 1000, 3

    def depth(self, d: int):
        if d not in (18, 34, 50):
            raise ValueError("depth must be 18, 34 or 50")
        self._depth = d
        return self

    def num_classes(self, n: int):
        self._classes = n
        return self

    def in_channels(self, c: int):
        self._in = c
        return self

    def build(self) -> ResNet:
        return {18: resnet18, 34: resnet34, 50: resnet50}[self._depth](self._classes, in_channels=self._in)
