"""Small building blocks shared by the CIFAR architectures."""
import torch.nn as nn


def conv_bn(cin: int, cout: int, k: int, stride: int = 1, groups: int = 1, padding=None):
    """A bias-free convolution and its BatchNorm (returned as a pair, named by the caller)."""
    pad = k // 2 if padding is None else padding
    return nn.Conv2d(cin, cout, kernel_size=k, stride=stride, padding=pad, groups=groups, bias=False), nn.BatchNorm2d(cout)
