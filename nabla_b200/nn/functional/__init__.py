"""Functional layers, losses, initialisers, and the activations re-exported from ``ops``
(reference: nabla/nn/functional/__init__.py)."""
from ...ops.unary import gelu, relu, sigmoid, silu, softmax, tanh
from .init import he_normal, xavier_normal
from .layers import (dropout, embedding, layer_norm, layer_norm_reference, linear, scaled_dot_product_attention,
                     scaled_dot_product_attention_reference, use_fused)
from .losses import cross_entropy_loss, cross_entropy_loss_reference, mse_loss
