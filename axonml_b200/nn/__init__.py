"""Neural-network modules with the reference's names and constructor shapes
(crates/axonml-nn)."""
from . import functional, init
from .init import (InitMode, constant, diag, eye, glorot_normal, glorot_uniform, he_normal, he_uniform, kaiming_normal,
                   kaiming_uniform, normal, ones, orthogonal, randn, sparse, uniform, uniform_range, xavier_normal, xavier_uniform,
                   zeros)
from .activation import (ELU, GELU, Identity, LeakyReLU, LogSoftmax, ReLU, Sigmoid, SiLU, Softmax,
                         Tanh)
from .layers import (GRU, LSTM, RNN, AdaptiveAvgPool2d, AlphaDropout, AvgPool1d, AvgPool2d,
                     BatchNorm1d, BatchNorm2d, Conv1d, Conv2d, Dropout, Dropout2d, Embedding,
                     GroupNorm, GRUCell, InstanceNorm2d, LayerNorm, Linear, LSTMCell, MaxPool1d,
                     MaxPool2d, MultiHeadAttention, RMSNorm, RNNCell)
from .loss import (BCELoss, BCEWithLogitsLoss, CrossEntropyLoss, L1Loss, MSELoss, NLLLoss,
                   Reduction, SmoothL1Loss)
from .module import Module, ModuleList, Parameter, Sequential

F = functional
