"""VGG-11/13/16/19 with optional BatchNorm (crates/axonml-vision/src/models/vgg.rs)."""
from __future__ import annotations

from ... import nn

_CFG = {11: [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
        13: [64, 64, "M", 128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
        16: [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"],
        19: [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"]}


class VGG(nn.Module):
    def __init__(self, depth: int = 16, num_classes: int = 1000, batch_norm: bool = False, in_channels: int = 3):
        super().__init__()
        layers, c = nn.Sequential(), in_channels
        for v in _CFG[depth]:
            if v == "M":
                layers.add(nn.MaxPool2d(2))
            else:
                layers.add(nn.Conv2d(c, v, 3, padding=1))
                if batch_norm:
                    layers.add(nn.BatchNorm2d(v))
                layers.add(nn.ReLU())
                c = v
        self.features = layers
        self.avgpool = nn.AdaptiveAvgPool2d((7, 7))
        self.classifier = nn.Sequential(nn.Linear(512 * 49, 4096), nn.ReLU(), nn.Dropout(0.5),
                                        nn.Linear(4096, 4096), nn.ReLU(), nn.Dropout(0.5), nn.Linear(4096, num_classes))

    def forward(self, x):
        return self.classifier(self.avgpool(self.features(x)).flatten(1))


def vgg11(num_classes=1000): return VGG(11, num_classes)
def vgg13(num_classes=1000): return VGG(13, num_classes)
def vgg16(num_classes=1000): return VGG(16, num_classes)
def vgg19(num_classes=1000): return VGG(19, num_classes)
def vgg11_bn(num_classes=1000): return VGG(11, num_classes, True)
def vgg13_bn(num_classes=1000): return VGG(13, num_classes, True)
def vgg16_bn(num_classes=1000): return VGG(16, num_classes, True)
def vgg19_bn(num_classes=1000): return VGG(19, num_classes, True)
