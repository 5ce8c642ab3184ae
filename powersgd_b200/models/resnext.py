"""ResNeXt-29 (three stages of three grouped-convolution bottlenecks, widths doubling).

Parity with paper-code/tasks/cifar_architectures/resnext.py:13-92, including the 1x1 stem.
"""
import torch.nn as nn
import torch.nn.functional as F

from ._blocks import conv_bn


class Block(nn.Module):
    expansion = 2

    def __init__(self, in_planes: int, cardinality: int = 32, bottleneck_width: int = 4, stride: int = 1):
        super().__init__()
        width = cardinality * bottleneck_width
        self.conv1, self.bn1 = conv_bn(in_planes, width, 1)
        self.conv2, self.bn2 = conv_bn(width, width, 3, stride, groups=cardinality)
        self.conv3, self.bn3 = conv_bn(width, self.expansion * width, 1)
        self.shortcut = nn.Sequential()
        if stride != 1 or in_planes != self.expansion * width:
            self.shortcut = nn.Sequential(*conv_bn(in_planes, self.expansion * width, 1, stride))

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = F.relu(self.bn2(self.conv2(y)))
        y = self.bn3(self.conv3(y))
        return F.relu(y + self.shortcut(x))


class ResNeXt(nn.Module):
    def __init__(self, num_blocks, cardinality: int, bottleneck_width: int, num_classes: int = 10):
        super().__init__()
        self.conv1, self.bn1 = conv_bn(3, 64, 1)
        in_planes, width = 64, bottleneck_width
        for i, (count, stride) in enumerate(zip(num_blocks, (1, 2, 2)), start=1):
            stage = []
            for s in [stride] + [1] * (count - 1):
                stage.append(Block(in_planes, cardinality, width, s))
                in_planes = Block.expansion * cardinality * width
            setattr(self, f"layer{i}", nn.Sequential(*stage))
            width *= 2  # the bottleneck widens after every stage
        self.linear = nn.Linear(cardinality * bottleneck_width * 8, num_classes)

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.layer3(self.layer2(self.layer1(y)))
        return self.linear(F.avg_pool2d(y, 8).flatten(1))


def ResNeXt29_2x64d(): return ResNeXt([3, 3, 3], cardinality=2, bottleneck_width=64)    # noqa: E704
def ResNeXt29_4x64d(): return ResNeXt([3, 3, 3], cardinality=4, bottleneck_width=64)    # noqa: E704
def ResNeXt29_8x64d(): return ResNeXt([3, 3, 3], cardinality=8, bottleneck_width=64)    # noqa: E704
def ResNeXt29_32x4d(): return ResNeXt([3, 3, 3], cardinality=32, bottleneck_width=4)    # noqa: E704
