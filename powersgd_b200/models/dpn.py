"""Dual-path networks: every block adds to a residual path and appends to a dense path.

Parity with paper-code/tasks/cifar_architectures/dpn.py:10-95 (grouped 3x3 with 32 groups).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ._blocks import conv_bn


class Bottleneck(nn.Module):
    def __init__(self, last_planes, in_planes, out_planes, dense_depth, stride, first_layer):
        super().__init__()
        self.out_planes, self.dense_depth = out_planes, dense_depth
        self.conv1, self.bn1 = conv_bn(last_planes, in_planes, 1)
        self.conv2, self.bn2 = conv_bn(in_planes, in_planes, 3, stride, groups=32)
        self.conv3, self.bn3 = conv_bn(in_planes, out_planes + dense_depth, 1)
        self.shortcut = nn.Sequential()
        if first_layer:
            self.shortcut = nn.Sequential(*conv_bn(last_planes, out_planes + dense_depth, 1, stride))

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = F.relu(self.bn2(self.conv2(y)))
        y = self.bn3(self.conv3(y))
        x = self.shortcut(x)
        d = self.out_planes
        return F.relu(torch.cat([x[:, :d] + y[:, :d], x[:, d:], y[:, d:]], 1))


class DPN(nn.Module):
    def __init__(self, cfg, num_classes: int = 10):
        super().__init__()
        self.conv1, self.bn1 = conv_bn(3, 64, 3)
        last = 64
        stages = zip(cfg["in_planes"], cfg["out_planes"], cfg["num_blocks"], cfg["dense_depth"], (1, 2, 2, 2))
        for i, (inp, out, count, depth, stride) in enumerate(stages, start=1):
            blocks = []
            for j, s in enumerate([stride] + [1] * (count - 1)):
                blocks.append(Bottleneck(last, inp, out, depth, s, j == 0))
                last = out + (j + 2) * depth
            setattr(self, f"layer{i}", nn.Sequential(*blocks))
        self.linear = nn.Linear(cfg["out_planes"][3] + (cfg["num_blocks"][3] + 1) * cfg["dense_depth"][3], num_classes)

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.layer4(self.layer3(self.layer2(self.layer1(y))))
        return self.linear(F.avg_pool2d(y, 4).flatten(1))


_COMMON = dict(in_planes=(96, 192, 384, 768), out_planes=(256, 512, 1024, 2048), dense_depth=(16, 32, 24, 128))


def DPN26():
    return DPN(dict(_COMMON, num_blocks=(2, 2, 2, 2)))


def DPN92():
    return DPN(dict(_COMMON, num_blocks=(3, 4, 20, 3)))
