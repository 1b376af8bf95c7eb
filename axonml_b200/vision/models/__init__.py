from .lenet import MLP, LeNet, SimpleCNN
from .resnet import BasicBlock, Bottleneck, ResNet, resnet18, resnet34, resnet50
from .transformer import (PositionalEncoding, Transformer, TransformerDecoder, TransformerDecoderLayer, TransformerEncoder,
                          TransformerEncoderLayer, VisionTransformer, vit_base, vit_large)
from .vgg import (VGG, VggClassifier, VggFeatures, VggLayer, vgg11, vgg11_bn, vgg11_config, vgg13, vgg13_bn, vgg13_config, vgg16,
                  vgg16_bn, vgg16_config, vgg19, vgg19_bn, vgg19_config)
