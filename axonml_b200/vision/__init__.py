"""Vision models, datasets and transforms (crates/axonml-vision)."""
from . import models
from .models import (MLP, BasicBlock, Bottleneck, LeNet, ResNet, SimpleCNN, resnet18, resnet34,
                     resnet50)
from . import datasets, transforms
from .datasets import (CIFAR10, CIFAR100, MNIST, FashionMNIST, SyntheticCIFAR, SyntheticImageNet, SyntheticMNIST)
from .models import (VGG, PositionalEncoding, Transformer, TransformerDecoder, TransformerEncoder, VggClassifier, VggFeatures,
                     VggLayer, VisionTransformer, vgg11, vgg11_bn, vgg11_config, vgg13, vgg13_bn, vgg13_config, vgg16, vgg16_bn,
                     vgg16_config, vgg19, vgg19_bn, vgg19_config, vit_base, vit_large)
from .transforms import (CenterCrop, ColorJitter, Grayscale, ImageNormalize, Pad, RandomHorizontalFlip,
                         RandomRotation, RandomVerticalFlip, Resize, ToTensorImage)
from . import hub
from .hub import (HubError, PretrainedModel, cache_dir, cached_path, download_weights, is_cached, list_models,
                  load_state_dict, model_info, model_registry, save_state_dict)
from ..serialize.state_dict import StateDict
