"""MobileNet v1 and v2, CIFAR variants (stride-1 stem).

Parity with paper-code/tasks/cifar_architectures/mobilenet.py:12-52 and mobilenetv2.py:13-77:
parameter names `conv1/bn1`, `layers.{i}.conv{1,2,3}/bn{1,2,3}/shortcut`, `conv2/bn2`, `linear`.
"""
import torch.nn as nn
import torch.nn.functional as F

from ._blocks import conv_bn


class _DepthwiseSeparable(nn.Module):
    def __init__(self, cin: int, cout: int, stride: int = 1):
        super().__init__()
        self.conv1, self.bn1 = conv_bn(cin, cin, 3, stride, groups=cin)
        self.conv2, self.bn2 = conv_bn(cin, cout, 1)

    def forward(self, x):
        x = F.relu(self.bn1(self.conv1(x)))
        return F.relu(self.bn2(self.conv2(x)))


class MobileNet(nn.Module):
    # an int is an output width at stride 1; a pair is (width, stride)
    cfg = [64, (128, 2), 128, (256, 2), 256, (512, 2), 512, 512, 512, 512, 512, (1024, 2), 1024]

    def __init__(self, num_classes: int = 10):
        super().__init__()
        self.conv1, self.bn1 = conv_bn(3, 32, 3)
        blocks, width = [], 32
        for item in self.cfg:
            out, stride = (item, 1) if isinstance(item, int) else item
            blocks.append(_DepthwiseSeparable(width, out, stride))
            width = out
        self.layers = nn.Sequential(*blocks)
        self.linear = nn.Linear(1024, num_classes)

    def forward(self, x):
        x = self.layers(F.relu(self.bn1(self.conv1(x))))
        return self.linear(F.avg_pool2d(x, 2).flatten(1))


class _InvertedResidual(nn.Module):
    def __init__(self, cin: int, cout: int, expansion: int, stride: int):
        super().__init__()
        self.stride = stride
        mid = expansion * cin
        self.conv1, self.bn1 = conv_bn(cin, mid, 1)
        self.conv2, self.bn2 = conv_bn(mid, mid, 3, stride, groups=mid)
        self.conv3, self.bn3 = conv_bn(mid, cout, 1)
        self.shortcut = nn.Sequential()
        if stride == 1 and cin != cout:
            self.shortcut = nn.Sequential(*conv_bn(cin, cout, 1))

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = F.relu(self.bn2(self.conv2(y)))
        y = self.bn3(self.conv3(y))
        return y + self.shortcut(x) if self.stride == 1 else y


class MobileNetV2(nn.Module):
    # (expansion, width, blocks, stride); the second stage keeps stride 1 for 32 x 32 inputs
    cfg = [(1, 16, 1, 1), (6, 24, 2, 1), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]

    def __init__(self, num_classes: int = 10):
        super().__init__()
        self.conv1, self.bn1 = conv_bn(3, 32, 3)
        blocks, width = [], 32
        for expansion, out, count, stride in self.cfg:
            for s in [stride] + [1] * (count - 1):
                blocks.append(_InvertedResidual(width, out, expansion, s))
                width = out
        self.layers = nn.Sequential(*blocks)
        self.conv2, self.bn2 = conv_bn(320, 1280, 1)
        self.linear = nn.Linear(1280, num_classes)

    def forward(self, x):
        x = self.layers(F.relu(self.bn1(self.conv1(x))))
        x = F.relu(self.bn2(self.conv2(x)))
        return self.linear(F.avg_pool2d(x, 4).flatten(1))
