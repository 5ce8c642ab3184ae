"""ShuffleNet (grouped 1x1 convolutions with a channel shuffle between them).

Parity with paper-code/tasks/cifar_architectures/shufflenet.py:13-104. The original divides
channel counts with `/` (a float under Python 3, which current PyTorch rejects); integer
division gives the intended widths.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ._blocks import conv_bn


class ShuffleBlock(nn.Module):
    def __init__(self, groups: int):
        super().__init__()
        self.groups = groups

    def forward(self, x):
        n, c, h, w = x.shape
        g = self.groups
        return x.view(n, g, c // g, h, w).transpose(1, 2).reshape(n, c, h, w)


class Bottleneck(nn.Module):
    def __init__(self, in_planes: int, out_planes: int, stride: int, groups: int):
        super().__init__()
        self.stride = stride
        mid = out_planes // 4
        g = 1 if in_planes == 24 else groups
        self.conv1, self.bn1 = conv_bn(in_planes, mid, 1, groups=g)
        self.shuffle1 = ShuffleBlock(groups=g)
        self.conv2, self.bn2 = conv_bn(mid, mid, 3, stride, groups=mid)
        self.conv3, self.bn3 = conv_bn(mid, out_planes, 1, groups=groups)
        self.shortcut = nn.Sequential(nn.AvgPool2d(3, stride=2, padding=1)) if stride == 2 else nn.Sequential()

    def forward(self, x):
        y = self.shuffle1(F.relu(self.bn1(self.conv1(x))))
        y = F.relu(self.bn2(self.conv2(y)))
        y = self.bn3(self.conv3(y))
        res = self.shortcut(x)
        return F.relu(torch.cat([y, res], 1)) if self.stride == 2 else F.relu(y + res)


class ShuffleNet(nn.Module):
    def __init__(self, cfg, num_classes: int = 10):
        super().__init__()
        self.conv1, self.bn1 = conv_bn(3, 24, 1)
        width = 24
        for i, (out, count) in enumerate(zip(cfg["out_planes"], cfg["num_blocks"]), start=1):
            blocks = []
            for j in range(count):
                # the first block of a stage halves the resolution and concatenates its input
                blocks.append(Bottleneck(width, out - (width if j == 0 else 0), stride=2 if j == 0 else 1, groups=cfg["groups"]))
                width = out
            setattr(self, f"layer{i}", nn.Sequential(*blocks))
        self.linear = nn.Linear(cfg["out_planes"][2], num_classes)

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.layer3(self.layer2(self.layer1(y)))
        return self.linear(F.avg_pool2d(y, 4).flatten(1))


def ShuffleNetG2():
    return ShuffleNet({"out_planes": [200, 400, 800], "num_blocks": [4, 8, 4], "groups": 2})


def ShuffleNetG3():
    return ShuffleNet({"out_planes": [240, 480, 960], "num_blocks": [4, 8, 4], "groups": 3})
