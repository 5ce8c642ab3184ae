"""VGG 11/13/16/19 with and without BatchNorm, CIFAR classifier head (512-512-10 with dropout).

Parity with paper-code/tasks/cifar_architectures/vgg.py:13-105: `features` / `classifier`
sub-modules, He-normal convolution weights with zero bias.
"""
import math

import torch.nn as nn

_PLANS = {
    11: [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
    13: [64, 64, "M", 128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
    16: [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"],
    19: [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"],
}


def make_layers(plan, batch_norm: bool = False) -> nn.Sequential:
    layers, channels = [], 3
    for item in plan:
        if item == "M":
            layers.append(nn.MaxPool2d(kernel_size=2, stride=2))
            continue
        layers.append(nn.Conv2d(channels, item, kernel_size=3, padding=1))
        if batch_norm:
            layers.append(nn.BatchNorm2d(item))
        layers.append(nn.ReLU(inplace=True))
        channels = item
    return nn.Sequential(*layers)


class VGG(nn.Module):
    def __init__(self, features: nn.Sequential, num_classes: int = 10):
        super().__init__()
        self.features = features
        self.classifier = nn.Sequential(
            nn.Dropout(), nn.Linear(512, 512), nn.ReLU(True), nn.Dropout(), nn.Linear(512, 512), nn.ReLU(True),
            nn.Linear(512, num_classes),
        )
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                fan = m.kernel_size[0] * m.kernel_size[1] * m.out_channels
                nn.init.normal_(m.weight, 0.0, math.sqrt(2.0 / fan))
                nn.init.zeros_(m.bias)

    def forward(self, x):
        return self.classifier(self.features(x).flatten(1))


def _build(depth: int, bn: bool) -> VGG:
    return VGG(make_layers(_PLANS[depth], batch_norm=bn))


def vgg11(): return _build(11, False)      # noqa: E704
def vgg11_bn(): return _build(11, True)    # noqa: E704
def vgg13(): return _build(13, False)      # noqa: E704
def vgg13_bn(): return _build(13, True)    # noqa: E704
def vgg16(): return _build(16, False)      # noqa: E704
def vgg16_bn(): return _build(16, True)    # noqa: E704
def vgg19(): return _build(19, False)      # noqa: E704
def vgg19_bn(): return _build(19, True)    # noqa: E704
