from .lenet import MLP, LeNet, SimpleCNN
from .resnet import BasicBlock, Bottleneck, ResNet, resnet18, resnet34, resnet50
