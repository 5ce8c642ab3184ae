"""Squeeze-and-excitation ResNet-18 (pre-activation blocks gated by a 1/16 bottleneck).

Parity with paper-code/tasks/cifar_architectures/senet.py:13-117 (`fc1`/`fc2` are 1x1
convolutions; `SENet18` uses the pre-activation block).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ._blocks import conv_bn


class _Gate(nn.Module):
    def _make_gate(self, planes: int) -> None:
        self.fc1 = nn.Conv2d(planes, planes // 16, kernel_size=1)
        self.fc2 = nn.Conv2d(planes // 16, planes, kernel_size=1)

    def _gate(self, y: torch.Tensor) -> torch.Tensor:
        w = F.adaptive_avg_pool2d(y, 1)
        return y * torch.sigmoid(self.fc2(F.relu(self.fc1(w))))


class BasicBlock(_Gate):
    def __init__(self, in_planes: int, planes: int, stride: int = 1):
        super().__init__()
        self.conv1, self.bn1 = conv_bn(in_planes, planes, 3, stride)
        self.conv2, self.bn2 = conv_bn(planes, planes, 3)
        self.shortcut = nn.Sequential()
        if stride != 1 or in_planes != planes:
            self.shortcut = nn.Sequential(*conv_bn(in_planes, planes, 1, stride, padding=0))
        self._make_gate(planes)

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = self._gate(self.bn2(self.conv2(y)))
        return F.relu(y + self.shortcut(x))


class PreActBlock(_Gate):
    def __init__(self, in_planes: int, planes: int, stride: int = 1):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(in_planes)
        self.conv1 = nn.Conv2d(in_planes, planes, 3, stride, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, 1, 1, bias=False)
        self.shortcut = None
        if stride != 1 or in_planes != planes:
            self.shortcut = nn.Sequential(nn.Conv2d(in_planes, planes, 1, stride, bias=False))
        self._make_gate(planes)

    def forward(self, x):
        pre = F.relu(self.bn1(x))
        skip = self.shortcut(pre) if self.shortcut is not None else x
        y = self.conv2(F.relu(self.bn2(self.conv1(pre))))
        return self._gate(y) + skip


class SENet(nn.Module):
    def __init__(self, block, num_blocks, num_classes: int = 10):
        super().__init__()
        self.conv1, self.bn1 = conv_bn(3, 64, 3)
        width = 64
        for i, (planes, stride, count) in enumerate(zip((64, 128, 256, 512), (1, 2, 2, 2), num_blocks), start=1):
            stage = []
            for s in [stride] + [1] * (count - 1):
                stage.append(block(width, planes, s))
                width = planes
            setattr(self, f"layer{i}", nn.Sequential(*stage))
        self.linear = nn.Linear(512, num_classes)

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.layer4(self.layer3(self.layer2(self.layer1(y))))
        return self.linear(F.avg_pool2d(y, 4).flatten(1))


def SENet18():
    return SENet(PreActBlock, [2, 2, 2, 2])
