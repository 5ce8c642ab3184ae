"""Pre-activation ResNets (BN-ReLU before each convolution; no BN on the shortcut).

Parity with paper-code/tasks/cifar_architectures/preact_resnet.py:14-115.
"""
import torch.nn as nn
import torch.nn.functional as F


def _plain_conv(cin, cout, k, stride=1):
    return nn.Conv2d(cin, cout, kernel_size=k, stride=stride, padding=k // 2, bias=False)


class PreActBlock(nn.Module):
    expansion = 1

    def __init__(self, in_planes: int, planes: int, stride: int = 1):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(in_planes)
        self.conv1 = _plain_conv(in_planes, planes, 3, stride)
        self.bn2 = nn.BatchNorm2d(planes)
        self.conv2 = _plain_conv(planes, planes, 3)
        self.shortcut = None
        if stride != 1 or in_planes != self.expansion * planes:
            self.shortcut = nn.Sequential(_plain_conv(in_planes, self.expansion * planes, 1, stride))

    def forward(self, x):
        pre = F.relu(self.bn1(x))
        skip = self.shortcut(pre) if self.shortcut is not None else x
        y = self.conv1(pre)
        y = self.conv2(F.relu(self.bn2(y)))
        return y + skip


class PreActBottleneck(nn.Module):
    expansion = 4

    def __init__(self, in_planes: int, planes: int, stride: int = 1):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(in_planes)
        self.conv1 = _plain_conv(in_planes, planes, 1)
        self.bn2 = nn.BatchNorm2d(planes)
        self.conv2 = _plain_conv(planes, planes, 3, stride)
        self.bn3 = nn.BatchNorm2d(planes)
        self.conv3 = _plain_conv(planes, self.expansion * planes, 1)
        self.shortcut = None
        if stride != 1 or in_planes != self.expansion * planes:
            self.shortcut = nn.Sequential(_plain_conv(in_planes, self.expansion * planes, 1, stride))

    def forward(self, x):
        pre = F.relu(self.bn1(x))
        skip = self.shortcut(pre) if self.shortcut is not None else x
        y = self.conv1(pre)
        y = self.conv2(F.relu(self.bn2(y)))
        y = self.conv3(F.relu(self.bn3(y)))
        return y + skip


class PreActResNet(nn.Module):
    def __init__(self, block, num_blocks, num_classes: int = 10):
        super().__init__()
        self.in_planes = 64
        self.conv1 = _plain_conv(3, 64, 3)
        for i, (planes, stride, count) in enumerate(zip((64, 128, 256, 512), (1, 2, 2, 2), num_blocks), start=1):
            stage = []
            for s in [stride] + [1] * (count - 1):
                stage.append(block(self.in_planes, planes, s))
                self.in_planes = planes * block.expansion
            setattr(self, f"layer{i}", nn.Sequential(*stage))
        self.linear = nn.Linear(512 * block.expansion, num_classes)

    def forward(self, x):
        y = self.layer4(self.layer3(self.layer2(self.layer1(self.conv1(x)))))
        return self.linear(F.avg_pool2d(y, 4).flatten(1))


def PreActResNet18(): return PreActResNet(PreActBlock, [2, 2, 2, 2])          # noqa: E704
def PreActResNet34(): return PreActResNet(PreActBlock, [3, 4, 6, 3])          # noqa: E704
def PreActResNet50(): return PreActResNet(PreActBottleneck, [3, 4, 6, 3])     # noqa: E704
def PreActResNet101(): return PreActResNet(PreActBottleneck, [3, 4, 23, 3])   # noqa: E704
def PreActResNet152(): return PreActResNet(PreActBottleneck, [3, 8, 36, 3])   # noqa: E704
