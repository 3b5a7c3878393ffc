"""Layers, losses and initialisers (ferrum-nn)."""
from . import init
from .loss import (bce_loss, cross_entropy, cross_entropy_loss, l1_loss, log_softmax, mse_loss, nll_loss,
                   smooth_l1_loss, softmax)
from .modules import (ELU, GELU, BatchNorm1d, Dropout, Embedding, LayerNorm, LeakyReLU, Linear, LogSoftmax,
                      MeanPoolEmbedding, Module, ReLU, Sequential, Sigmoid, SiLU, Softmax, Tanh, tensor_io)

__all__ = [
    "Module", "Linear", "Sequential", "ReLU", "Sigmoid", "Tanh", "GELU", "SiLU", "LeakyReLU", "ELU", "Softmax",
    "LogSoftmax", "LayerNorm", "BatchNorm1d", "Dropout", "Embedding", "MeanPoolEmbedding", "mse_loss", "bce_loss",
    "l1_loss", "smooth_l1_loss", "cross_entropy_loss", "nll_loss", "cross_entropy", "softmax", "log_softmax",
    "init", "tensor_io",
]
