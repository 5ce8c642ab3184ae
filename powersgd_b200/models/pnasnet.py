"""PNASNet-style cell networks (cells A and B; depthwise 'separable' convolutions + BN).

Parity with paper-code/tasks/cifar_architectures/pnasnet.py:13-128: `conv1/bn1`,
`layer1..layer5` (6 cells, downsample, 6 cells, downsample, 6 cells), `linear`.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ._blocks import conv_bn


class SepConv(nn.Module):
    def __init__(self, in_planes: int, out_planes: int, kernel_size: int, stride: int):
        super().__init__()
        self.conv1, self.bn1 = conv_bn(in_planes, out_planes, kernel_size, stride, groups=in_planes)

    def forward(self, x):
        return self.bn1(self.conv1(x))


class _Cell(nn.Module):
    def _pooled(self, x):
        y = F.max_pool2d(x, kernel_size=3, stride=self.stride, padding=1)
        return self.bn1(self.conv1(y)) if self.stride == 2 else y


class CellA(_Cell):
    def __init__(self, in_planes: int, out_planes: int, stride: int = 1):
        super().__init__()
        self.stride = stride
        self.sep_conv1 = SepConv(in_planes, out_planes, 7, stride)
        if stride == 2:
            self.conv1, self.bn1 = conv_bn(in_planes, out_planes, 1)

    def forward(self, x):
        return F.relu(self.sep_conv1(x) + self._pooled(x))


class CellB(_Cell):
    def __init__(self, in_planes: int, out_planes: int, stride: int = 1):
        super().__init__()
        self.stride = stride
        self.sep_conv1 = SepConv(in_planes, out_planes, 7, stride)
        self.sep_conv2 = SepConv(in_planes, out_planes, 3, stride)
        self.sep_conv3 = SepConv(in_planes, out_planes, 5, stride)
        if stride == 2:
            self.conv1, self.bn1 = conv_bn(in_planes, out_planes, 1)
        self.conv2, self.bn2 = conv_bn(2 * out_planes, out_planes, 1)

    def forward(self, x):
        left = F.relu(self.sep_conv1(x) + self.sep_conv2(x))
        right = F.relu(self._pooled(x) + self.sep_conv3(x))
        return F.relu(self.bn2(self.conv2(torch.cat([left, right], 1))))


class PNASNet(nn.Module):
    def __init__(self, cell_type, num_cells: int, num_planes: int, num_classes: int = 10):
        super().__init__()
        self.conv1, self.bn1 = conv_bn(3, num_planes, 3)
        width = num_planes

        def stack(planes):
            nonlocal width
            cells = []
            for _ in range(num_cells):
                cells.append(cell_type(width, planes, stride=1))
                width = planes
            return nn.Sequential(*cells)

        def down(planes):
            nonlocal width
            cell = cell_type(width, planes, stride=2)
            width = planes
            return cell

        self.layer1 = stack(num_planes)
        self.layer2 = down(num_planes * 2)
        self.layer3 = stack(num_planes * 2)
        self.layer4 = down(num_planes * 4)
        self.layer5 = stack(num_planes * 4)
        self.linear = nn.Linear(num_planes * 4, num_classes)

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.layer5(self.layer4(self.layer3(self.layer2(self.layer1(y)))))
        return self.linear(F.avg_pool2d(y, 8).flatten(1))


def PNASNetA():
    return PNASNet(CellA, num_cells=6, num_planes=44)


def PNASNetB():
    return PNASNet(CellB, num_cells=6, num_planes=32)
