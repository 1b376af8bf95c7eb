"""Vision models, datasets and transforms (crates/axonml-vision)."""
from . import models
from .models import (MLP, BasicBlock, Bottleneck, LeNet, ResNet, SimpleCNN, resnet18, resnet34,
                     resnet50)
