from . import finetune, functional, optim
from .functional import (cross_entropy_loss, dropout, embedding, he_normal, layer_norm, linear, mse_loss,
                         scaled_dot_product_attention, xavier_normal)
from .modules import (GELU, Dropout, Embedding, LayerNorm, Linear, Module, MultiHeadAttention, ReLU, Sequential,
                      Sigmoid, SiLU, Softmax, Tanh, TransformerDecoderLayer, TransformerEncoderLayer)
from .optim import SGD, AdamW, Optimizer, adamw_init, adamw_step, adamw_update, sgd_step, sgd_update
