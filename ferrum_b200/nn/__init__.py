"""Layers, losses and initialisers (ferrum-nn)."""
from . import init
from .loss import (bce_loss, cross_entropy, cross_entropy_loss, l1_loss, log_softmax, mse_loss, nll_loss,
                   smooth_l1_loss, softmax)
from .conv import AdaptiveAvgPool2d, AvgPool2d, Conv1d, Conv2d, MaxPool2d
from .rnn import GRU, LSTM, RNN, GRUCell, LSTMCell, Nonlinearity, RNNCell
from .transformer import MultiHeadAttention, PositionalEncoding, TransformerEncoderLayer
from .modules import (ELU, GELU, BatchNorm1d, Dropout, Embedding, LayerNorm, LeakyReLU, Linear, LogSoftmax,
                      MeanPoolEmbedding, Module, ReLU, Sequential, Sigmoid, SiLU, Softmax, Tanh, tensor_io)

__all__ = [
    "Module", "Linear", "Sequential", "ReLU", "Sigmoid", "Tanh", "GELU", "SiLU", "LeakyReLU", "ELU", "Softmax",
    "LogSoftmax", "LayerNorm", "BatchNorm1d", "Dropout", "Embedding", "MeanPoolEmbedding", "mse_loss", "bce_loss",
    "l1_loss", "smooth_l1_loss", "cross_entropy_loss", "nll_loss", "cross_entropy", "softmax", "log_softmax",
    "init", "tensor_io", "Conv1d", "Conv2d", "MaxPool2d", "AvgPool2d", "AdaptiveAvgPool2d", "RNNCell", "LSTMCell",
    "GRUCell", "RNN", "LSTM", "GRU", "Nonlinearity", "MultiHeadAttention", "TransformerEncoderLayer",
    "PositionalEncoding", "BasicBlock", "ResNet", "VGG", "MLP",
]

_ZOO = {"BasicBlock": "vision", "ResNet": "vision", "VGG": "vision", "MLP": "mlp"}


def __getattr__(name):
    # the model zoo sits in ferrum_b200.models (it imports this package); the reference exports it from its nn
    # crate (ferrum-nn/src/models.rs:13-284), so the names resolve here too, on first use
    if name in _ZOO:
        import importlib

        return getattr(importlib.import_module(f"..models.{_ZOO[name]}", __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
