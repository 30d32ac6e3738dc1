from .base import Module
from .layers import (GELU, Dropout, Embedding, LayerNorm, Linear, MultiHeadAttention, ReLU, Sequential, Sigmoid, SiLU,
                     Softmax, Tanh, TransformerDecoderLayer, TransformerEncoderLayer)
