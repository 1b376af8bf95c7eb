"""Vision models, datasets and transforms (crates/axonml-vision)."""
from . import models
from .models import (MLP, BasicBlock, Bottleneck, LeNet, ResNet, SimpleCNN, resnet18, resnet34,
                     resnet50)
from . import datasets, transforms
from .datasets import (CIFAR10, CIFAR100, MNIST, FashionMNIST, SyntheticCIFAR, SyntheticImageNet, SyntheticMNIST)
from .models import (VGG, Transformer, TransformerDecoder, TransformerEncoder, VisionTransformer, vgg11, vgg16,
                     vgg19)
from .transforms import (CenterCrop, ColorJitter, Grayscale, ImageNormalize, Pad, RandomHorizontalFlip,
                         RandomRotation, RandomVerticalFlip, Resize, ToTensorImage)
