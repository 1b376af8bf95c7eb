from .attention import MultiHeadAttention
from .conv import Conv1d, Conv2d
from .dropout import AlphaDropout, Dropout, Dropout2d
from .embedding import Embedding
from .linear import Linear
from .norm import (BatchNorm1d, BatchNorm2d, GroupNorm, InstanceNorm2d, LayerNorm, RMSNorm)
from .pooling import AdaptiveAvgPool2d, AvgPool1d, AvgPool2d, MaxPool1d, MaxPool2d
from .rnn import GRU, LSTM, RNN, GRUCell, LSTMCell, RNNCell
