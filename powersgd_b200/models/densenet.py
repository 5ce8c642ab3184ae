"""DenseNet-BC (bottleneck layers, 0.5 compression at the transitions).

Parity with paper-code/tasks/cifar_architectures/densenet.py:13-101: `conv1`, `dense{1..4}`,
`trans{1..3}`, `bn`, `linear`.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class Bottleneck(nn.Module):
    def __init__(self, in_planes: int, growth_rate: int):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(in_planes)
        self.conv1 = nn.Conv2d(in_planes, 4 * growth_rate, kernel_size=1, bias=False)
        self.bn2 = nn.BatchNorm2d(4 * growth_rate)
        self.conv2 = nn.Conv2d(4 * growth_rate, growth_rate, kernel_size=3, padding=1, bias=False)

    def forward(self, x):
        y = self.conv1(F.relu(self.bn1(x)))
        y = self.conv2(F.relu(self.bn2(y)))
        return torch.cat([y, x], 1)


class Transition(nn.Module):
    def __init__(self, in_planes: int, out_planes: int):
        super().__init__()
        self.bn = nn.BatchNorm2d(in_planes)
        self.conv = nn.Conv2d(in_planes, out_planes, kernel_size=1, bias=False)

    def forward(self, x):
        return F.avg_pool2d(self.conv(F.relu(self.bn(x))), 2)


class DenseNet(nn.Module):
    def __init__(self, block, nblocks, growth_rate: int = 12, reduction: float = 0.5, num_classes: int = 10):
        super().__init__()
        self.growth_rate = growth_rate
        planes = 2 * growth_rate
        self.conv1 = nn.Conv2d(3, planes, kernel_size=3, padding=1, bias=False)
        for i, count in enumerate(nblocks, start=1):
            layers = []
            for _ in range(count):
                layers.append(block(planes, growth_rate))
                planes += growth_rate
            setattr(self, f"dense{i}", nn.Sequential(*layers))
            if i < len(nblocks):
                out = int(math.floor(planes * reduction))
                setattr(self, f"trans{i}", Transition(planes, out))
                planes = out
        self.bn = nn.BatchNorm2d(planes)
        self.linear = nn.Linear(planes, num_classes)

    def forward(self, x):
        y = self.conv1(x)
        y = self.trans1(self.dense1(y))
        y = self.trans2(self.dense2(y))
        y = self.trans3(self.dense3(y))
        y = self.dense4(y)
        return self.linear(F.avg_pool2d(F.relu(self.bn(y)), 4).flatten(1))


def DenseNet121(): return DenseNet(Bottleneck, [6, 12, 24, 16], growth_rate=32)    # noqa: E704
def DenseNet169(): return DenseNet(Bottleneck, [6, 12, 32, 32], growth_rate=32)    # noqa: E704
def DenseNet201(): return DenseNet(Bottleneck, [6, 12, 48, 32], growth_rate=32)    # noqa: E704
def DenseNet161(): return DenseNet(Bottleneck, [6, 12, 36, 24], growth_rate=48)    # noqa: E704
def densenet_cifar(): return DenseNet(Bottleneck, [6, 12, 24, 16], growth_rate=12)  # noqa: E704
