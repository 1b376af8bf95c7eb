"""LeNet-5, SimpleCNN and MLP (crates/axonml-vision/src/models/lenet.rs:36-45 and siblings).
``LeNet.new()`` is the classic MNIST network: conv 1->6 5x5 pad 2, ReLU, maxpool 2; conv 6->16 5x5,
ReLU, maxpool 2; FC 400->120->84->10 (the reference builds conv1 without padding and therefore
256->120).  ``LeNet.for_cifar10()`` takes 3x32x32 inputs."""
from __future__ import annotations

import torch

from ... import nn


class LeNet(nn.Module):
    def __init__(self, in_channels: int = 1, num_classes: int = 10, input_size: int = 28):
        super().__init__()
        pad = 2 if input_size == 28 else 0
        self.conv1 = nn.Conv2d(in_channels, 6, 5, padding=pad)
        self.conv2 = nn.Conv2d(6, 16, 5)
        self.pool = nn.MaxPool2d(2)
        side = ((input_size + 2 * pad - 4) // 2 - 4) // 2
        self.fc1 = nn.Linear(16 * side * side, 120)
        self.fc2 = nn.Linear(120, 84)
        self.fc3 = nn.Linear(84, num_classes)
        self.relu = nn.ReLU()

    @classmethod
    def new(cls): return cls()

    @classmethod
    def for_cifar10(cls): return cls(3, 10, 32)

    def forward(self, x):
        if x.dim() == 3:
            x = x.unsqueeze(1)
        x = self.pool(self.relu(self.conv1(x)))
        x = self.pool(self.relu(self.conv2(x)))
        x = x.flatten(1)
        return self.fc3(self.relu(self.fc2(self.relu(self.fc1(x)))))


class SimpleCNN(nn.Module):
    def __init__(self, in_channels: int = 1, num_classes: int = 10, input_size: int = 28):
        super().__init__()
        self.conv1 = nn.Conv2d(in_channels, 32, 3, padding=1)
        self.conv2 = nn.Conv2d(32, 64, 3, padding=1)
        self.pool = nn.MaxPool2d(2)
        self.relu = nn.ReLU()
        side = input_size // 4
        self.fc1 = nn.Linear(64 * side * side, 128)
        self.fc2 = nn.Linear(128, num_classes)
        self._in_channels, self._num_classes = in_channels, num_classes

    def input_channels(self) -> int: return self._in_channels
    def num_classes(self) -> int: return self._num_classes

    @classmethod
    def new(cls, in_channels=1, num_classes=10): return cls(in_channels, num_classes)

    @classmethod
    def for_mnist(cls): return cls(1, 10, 28)

    @classmethod
    def for_cifar10(cls): return cls(3, 10, 32)

    def forward(self, x):
        x = self.pool(self.relu(self.conv1(x)))
        x = self.pool(self.relu(self.conv2(x)))
        return self.fc2(self.relu(self.fc1(x.flatten(1))))


class MLP(nn.Module):
    def __init__(self, input_size: int, hidden_sizes, num_classes: int, dropout: float = 0.0):
        super().__init__()
        layers = nn.Sequential()
        prev = input_size
        for h in hidden_sizes:
            layers.add(nn.Linear(prev, h)).add(nn.ReLU())
            if dropout > 0:
                layers.add(nn.Dropout(dropout))
            prev = h
        layers.add(nn.Linear(prev, num_classes))
        self.layers = layers

    @classmethod
    def new(cls, input_size, hidden_sizes, num_classes): return cls(input_size, hidden_sizes, num_classes)

    @classmethod
    def for_mnist(cls): return cls(784, [256, 128], 10)

    @classmethod
    def for_cifar10(cls): return cls(3072, [512, 256], 10)

    def forward(self, x):
        return self.layers(x.flatten(1))
