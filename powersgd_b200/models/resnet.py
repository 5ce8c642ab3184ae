"""CIFAR-style residual networks (3x3 stem, no max-pool, 4x4 average pool, 10 classes).

Architecture parity with paper-code/tasks/cifar_architectures/resnet.py:16-121 (same layer
names, so parameter names — which drive the per-parameter weight-decay / learning-rate rules
of the training loop — match): `conv1/bn1`, `layer{1..4}.{i}.conv{1,2,3}/bn{1,2,3}/shortcut`,
`linear`. `use_batchnorm=False` replaces every BatchNorm by an identity.
"""
from __future__ import annotations

from typing import List, Type

import torch
import torch.nn as nn
import torch.nn.functional as F


def _norm(channels: int, enabled: bool) -> nn.Module:
    return nn.BatchNorm2d(channels) if enabled else nn.Sequential()


def _conv(cin: int, cout: int, k: int, stride: int = 1) -> nn.Conv2d:
    return nn.Conv2d(cin, cout, kernel_size=k, stride=stride, padding=k // 2, bias=False)


class _Residual(nn.Module):
    expansion = 1

    def _make_shortcut(self, cin: int, cout: int, stride: int, bn: bool) -> nn.Sequential:
        if stride == 1 and cin == cout:
            return nn.Sequential()
        return nn.Sequential(_conv(cin, cout, 1, stride), _norm(cout, bn))


class BasicBlock(_Residual):
    expansion = 1

    def __init__(self, in_planes: int, planes: int, stride: int = 1, use_batchnorm: bool = True):
        super().__init__()
        self.conv1 = _conv(in_planes, planes, 3, stride)
        self.bn1 = _norm(planes, use_batchnorm)
        self.conv2 = _conv(planes, planes, 3)
        self.bn2 = _norm(planes, use_batchnorm)
        self.shortcut = self._make_shortcut(in_planes, planes, stride, use_batchnorm)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.bn2(self.conv2(y))
        return F.relu(y + self.shortcut(x))


class Bottleneck(_Residual):
    expansion = 4

    def __init__(self, in_planes: int, planes: int, stride: int = 1, use_batchnorm: bool = True):
        super().__init__()
        wide = planes * self.expansion
        self.conv1 = _conv(in_planes, planes, 1)
        self.bn1 = _norm(planes, use_batchnorm)
        self.conv2 = _conv(planes, planes, 3, stride)
        self.bn2 = _norm(planes, use_batchnorm)
        self.conv3 = _conv(planes, wide, 1)
        self.bn3 = _norm(wide, use_batchnorm)
        self.shortcut = self._make_shortcut(in_planes, wide, stride, use_batchnorm)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = F.relu(self.bn1(self.conv1(x)))
        y = F.relu(self.bn2(self.conv2(y)))
        y = self.bn3(self.conv3(y))
        return F.relu(y + self.shortcut(x))


class ResNet(nn.Module):
    def __init__(self, block: Type[_Residual], num_blocks: List[int], num_classes: int = 10, use_batchnorm: bool = True):
        super().__init__()
        self.use_batchnorm = use_batchnorm
        self.in_planes = 64
        self.conv1 = _conv(3, 64, 3)
        self.bn1 = _norm(64, use_batchnorm)
        widths, strides = (64, 128, 256, 512), (1, 2, 2, 2)
        for i, (w, s, nb) in enumerate(zip(widths, strides, num_blocks), start=1):
            setattr(self, f"layer{i}", self._stage(block, w, nb, s))
        self.linear = nn.Linear(512 * block.expansion, num_classes)

    def _stage(self, block, planes: int, count: int, stride: int) -> nn.Sequential:
        blocks = []
        for s in [stride] + [1] * (count - 1):
            blocks.append(block(self.in_planes, planes, s, self.use_batchnorm))
            self.in_planes = planes * block.expansion
        return nn.Sequential(*blocks)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.layer4(self.layer3(self.layer2(self.layer1(y))))
        y = F.avg_pool2d(y, 4).flatten(1)
        return self.linear(y)


def ResNet18(use_batchnorm: bool = True) -> ResNet:
    return ResNet(BasicBlock, [2, 2, 2, 2], use_batchnorm=use_batchnorm)


def ResNet34(use_batchnorm: bool = True) -> ResNet:
    return ResNet(BasicBlock, [3, 4, 6, 3], use_batchnorm=use_batchnorm)


def ResNet50(use_batchnorm: bool = True) -> ResNet:
    return ResNet(Bottleneck, [3, 4, 6, 3], use_batchnorm=use_batchnorm)


def ResNet101(use_batchnorm: bool = True) -> ResNet:
    return ResNet(Bottleneck, [3, 4, 23, 3], use_batchnorm=use_batchnorm)


def ResNet152(use_batchnorm: bool = True) -> ResNet:
    return ResNet(Bottleneck, [3, 8, 36, 3], use_batchnorm=use_batchnorm)
