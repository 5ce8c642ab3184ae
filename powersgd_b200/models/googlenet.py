"""GoogLeNet (Inception v1 with BatchNorm; the 5x5 branch is two stacked 3x3 convolutions).

Parity with paper-code/tasks/cifar_architectures/googlenet.py:10-101: `pre_layers`, inception
modules `a3 b3 a4 b4 c4 d4 e4 a5 b5` with branches `b1..b4`, `linear`.
"""
import torch
import torch.nn as nn


def _unit(cin: int, cout: int, k: int):
    """Biased convolution + BatchNorm + ReLU, as a flat list of modules."""
    return [nn.Conv2d(cin, cout, kernel_size=k, padding=k // 2), nn.BatchNorm2d(cout), nn.ReLU(True)]


class Inception(nn.Module):
    def __init__(self, in_planes, n1x1, n3x3red, n3x3, n5x5red, n5x5, pool_planes):
        super().__init__()
        self.b1 = nn.Sequential(*_unit(in_planes, n1x1, 1))
        self.b2 = nn.Sequential(*_unit(in_planes, n3x3red, 1), *_unit(n3x3red, n3x3, 3))
        self.b3 = nn.Sequential(*_unit(in_planes, n5x5red, 1), *_unit(n5x5red, n5x5, 3), *_unit(n5x5, n5x5, 3))
        self.b4 = nn.Sequential(nn.MaxPool2d(3, stride=1, padding=1), *_unit(in_planes, pool_planes, 1))

    def forward(self, x):
        return torch.cat([self.b1(x), self.b2(x), self.b3(x), self.b4(x)], 1)


class GoogLeNet(nn.Module):
    _SPEC = [
        ("a3", (192, 64, 96, 128, 16, 32, 32)), ("b3", (256, 128, 128, 192, 32, 96, 64)),
        ("a4", (480, 192, 96, 208, 16, 48, 64)), ("b4", (512, 160, 112, 224, 24, 64, 64)),
        ("c4", (512, 128, 128, 256, 24, 64, 64)), ("d4", (512, 112, 144, 288, 32, 64, 64)),
        ("e4", (528, 256, 160, 320, 32, 128, 128)), ("a5", (832, 256, 160, 320, 32, 128, 128)),
        ("b5", (832, 384, 192, 384, 48, 128, 128)),
    ]

    def __init__(self, num_classes: int = 10):
        super().__init__()
        self.pre_layers = nn.Sequential(*_unit(3, 192, 3))
        for name, spec in self._SPEC:
            setattr(self, name, Inception(*spec))
        self.maxpool = nn.MaxPool2d(3, stride=2, padding=1)
        self.avgpool = nn.AvgPool2d(8, stride=1)
        self.linear = nn.Linear(1024, num_classes)

    def forward(self, x):
        y = self.b3(self.a3(self.pre_layers(x)))
        y = self.maxpool(y)
        y = self.e4(self.d4(self.c4(self.b4(self.a4(y)))))
        y = self.maxpool(y)
        y = self.b5(self.a5(y))
        return self.linear(self.avgpool(y).flatten(1))
