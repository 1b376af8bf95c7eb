"""ResNet-18 / ResNet-34 (crates/axonml-vision/src/models/resnet.rs): BasicBlock and Bottleneck,
constructors ``resnet18(num_classes)`` / ``resnet34(num_classes)``.  Convolutions in front of a
BatchNorm carry no bias (the reference builds them with a bias that BatchNorm cancels,
resnet.rs:74-84).  The model runs channels-last on CUDA."""
from __future__ import annotations

import torch

from ... import nn


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, inplanes: int, planes: int, stride: int = 1):
        super().__init__()
        self.conv1 = nn.Conv2d(inplanes, planes, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.relu = nn.ReLU()
        self.downsample = None
        if stride != 1 or inplanes != planes * self.expansion:
            self.downsample = nn.Sequential(nn.Conv2d(inplanes, planes * self.expansion, 1, stride, 0, bias=False),
                                            nn.BatchNorm2d(planes * self.expansion))

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = self.bn1(self.conv1(x), relu=True)
        return self.bn2(self.conv2(out), relu=True, residual=idt)       # relu(bn(conv) + identity), one pass


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes: int, planes: int, stride: int = 1):
        super().__init__()
        self.conv1 = nn.Conv2d(inplanes, planes, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, stride, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.conv3 = nn.Conv2d(planes, planes * 4, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(planes * 4)
        self.relu = nn.ReLU()
        self.downsample = None
        if stride != 1 or inplanes != planes * 4:
            self.downsample = nn.Sequential(nn.Conv2d(inplanes, planes * 4, 1, stride, 0, bias=False),
                                            nn.BatchNorm2d(planes * 4))

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = self.relu(self.bn1(self.conv1(x)))
        out = self.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        return self.relu(out + idt)


class ResNet(nn.Module):
    def __init__(self, block, layers, num_classes: int = 1000, in_channels: int = 3):
        super().__init__()
        self.inplanes = 64
        self.conv1 = nn.Conv2d(in_channels, 64, 7, 2, 3, bias=False)
        self.bn1 = nn.BatchNorm2d(64)
        self.relu = nn.ReLU()
        self.maxpool = nn.MaxPool2d(3, 2, 1)
        self.layer1 = self._make_layer(block, 64, layers[0], 1)
        self.layer2 = self._make_layer(block, 128, layers[1], 2)
        self.layer3 = self._make_layer(block, 256, layers[2], 2)
        self.layer4 = self._make_layer(block, 512, layers[3], 2)
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(512 * block.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                torch.nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def _make_layer(self, block, planes, blocks, stride):
        seq = nn.Sequential()
        seq.add(block(self.inplanes, planes, stride))
        self.inplanes = planes * block.expansion
        for _ in range(1, blocks):
            seq.add(block(self.inplanes, planes))
        return seq

    @classmethod
    def resnet18(cls, num_classes: int = 1000): return cls(BasicBlock, [2, 2, 2, 2], num_classes)

    @classmethod
    def resnet34(cls, num_classes: int = 1000): return cls(BasicBlock, [3, 4, 6, 3], num_classes)

    @classmethod
    def resnet50(cls, num_classes: int = 1000): return cls(Bottleneck, [3, 4, 6, 3], num_classes)

    def forward(self, x):
        x = self.maxpool(self.bn1(self.conv1(x), relu=True))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(self.avgpool(x).flatten(1))


def resnet18(num_classes: int = 1000) -> ResNet: return ResNet.resnet18(num_classes)
def resnet34(num_classes: int = 1000) -> ResNet: return ResNet.resnet34(num_classes)
def resnet50(num_classes: int = 1000) -> ResNet: return ResNet.resnet50(num_classes)
