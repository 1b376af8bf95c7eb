from .lenet import MLP, LeNet, SimpleCNN
from .resnet import BasicBlock, Bottleneck, ResNet, resnet18, resnet34, resnet50
from .transformer import (Transformer, TransformerDecoder, TransformerDecoderLayer, TransformerEncoder,
                          TransformerEncoderLayer, VisionTransformer)
from .vgg import VGG, vgg11, vgg11_bn, vgg13, vgg13_bn, vgg16, vgg16_bn, vgg19, vgg19_bn
