"""Neural-network modules with the reference's names and constructor shapes
(crates/axonml-nn)."""
from . import functional, init
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
