"""VGG-11/13/16/19 with optional BatchNorm (crates/axonml-vision/src/models/vgg.rs)."""
from __future__ import annotations

from ... import nn

_CFG = {11: [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
        13: [64, 64, "M", 128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
        16: [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"],
        19: [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"]}


class VggLayer:
    """One entry of a VGG layout (vgg.rs:52-57): ``VggLayer.Conv(channels)`` or ``VggLayer.MaxPool``."""

    def __init__(self, kind: str, channels: int = 0):
        self.kind, self.channels = kind, channels

    @classmethod
    def Conv(cls, channels: int): return cls("conv", int(channels))

    def is_pool(self) -> bool: return self.kind == "pool"
    def __eq__(self, other): return isinstance(other, VggLayer) and (self.kind, self.channels) == (other.kind, other.channels)
    def __hash__(self): return hash((self.kind, self.channels))
    def __repr__(self): return "MaxPool" if self.is_pool() else f"Conv({self.channels})"


VggLayer.MaxPool = VggLayer("pool")


def _config(depth: int) -> list:
    return [VggLayer.MaxPool if v == "M" else VggLayer.Conv(v) for v in _CFG[depth]]


def vgg11_config() -> list: return _config(11)
def vgg13_config() -> list: return _config(13)
def vgg16_config() -> list: return _config(16)
def vgg19_config() -> list: return _config(19)


class VggFeatures(nn.Sequential):
    """The convolutional trunk built from a layout: 3x3 convolutions with padding 1 (followed by
    BatchNorm when asked) and ReLU, 2x2 max pooling between the stages (vgg.rs:163-265)."""

    def __init__(self, config, batch_norm: bool = False, in_channels: int = 3):
        super().__init__()
        c = in_channels
        for layer in config:
            if layer.is_pool():
                self.add(nn.MaxPool2d(2))
            else:
                self.add(nn.Conv2d(c, layer.channels, 3, padding=1))
                if batch_norm:
                    self.add(nn.BatchNorm2d(layer.channels))
                self.add(nn.ReLU())
                c = layer.channels
        self.out_channels = c


class VggClassifier(nn.Sequential):
    """512*7*7 -> 4096 -> 4096 -> classes with ReLU and dropout 0.5 between (vgg.rs:269-330)."""

    def __init__(self, num_classes: int = 1000, in_features: int = 512 * 49, dropout: float = 0.5):
        super().__init__(nn.Linear(in_features, 4096), nn.ReLU(), nn.Dropout(dropout),
                         nn.Linear(4096, 4096), nn.ReLU(), nn.Dropout(dropout), nn.Linear(4096, num_classes))

    @classmethod
    def new(cls, num_classes: int): return cls(num_classes)

    @classmethod
    def with_input_size(cls, input_features: int, num_classes: int):
        """Classifier for a trunk whose flattened output has ``input_features`` values."""
        return cls(num_classes, input_features)


class VGG(nn.Module):
    def __init__(self, depth: int = 16, num_classes: int = 1000, batch_norm: bool = False, in_channels: int = 3):
        super().__init__()
        self.features = VggFeatures(_config(depth), batch_norm, in_channels)
        self.avgpool = nn.AdaptiveAvgPool2d((7, 7))
        self.classifier = VggClassifier(num_classes)

    def forward(self, x):
        return self.classifier(self.avgpool(self.features(x)).flatten(1))


# the constructors under the class as well (vgg.rs ``VGG::vgg11`` ... ``VGG::vgg19_bn``)
for _depth in (11, 13, 16, 19):
    setattr(VGG, f"vgg{_depth}", classmethod(lambda cls, num_classes=1000, _d=_depth: cls(_d, num_classes)))
    setattr(VGG, f"vgg{_depth}_bn", classmethod(lambda cls, num_classes=1000, _d=_depth: cls(_d, num_classes, True)))


def vgg11(num_classes=1000): return VGG(11, num_classes)
def vgg13(num_classes=1000): return VGG(13, num_classes)
def vgg16(num_classes=1000): return VGG(16, num_classes)
def vgg19(num_classes=1000): return VGG(19, num_classes)
def vgg11_bn(num_classes=1000): return VGG(11, num_classes, True)
def vgg13_bn(num_classes=1000): return VGG(13, num_classes, True)
def vgg16_bn(num_classes=1000): return VGG(16, num_classes, True)
def vgg19_bn(num_classes=1000): return VGG(19, num_classes, True)
