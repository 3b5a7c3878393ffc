"""Multi-layer perceptrons: the reference's ``MLP`` (ferrum-nn/src/models.rs:247-284, ReLU between
Linears) and the benchmark networks built from ``Linear -> GELU -> LayerNorm`` blocks."""
from __future__ import annotations

from .. import nn


class MLP(nn.Sequential):
    """``MLP([in, h1, ..., out])``: Linear layers with ReLU between them (none after the last)."""

    def __init__(self, layer_sizes, device=None):
        layers = []
        sizes = list(layer_sizes)
        for i in range(len(sizes) - 1):
            layers.append(nn.Linear(sizes[i], sizes[i + 1], device=device))
            if i < len(sizes) - 2:
                layers.append(nn.ReLU())
        super().__init__(*layers)
        self.layer_sizes = sizes

    @classmethod
    def new(cls, layer_sizes):
        return cls(layer_sizes)


def wide_mlp(in_features: int = 1024, width: int = 4096, depth: int = 8, num_classes: int = 1000,
             device=None) -> nn.Sequential:
    """``depth`` blocks of Linear(width) - GELU - LayerNorm(width) and a ``num_classes``-way head.

    With the defaults this is the 125.8 M-parameter network of the headline benchmark
    (1024 input features, 8 blocks of width 4096, 1000 classes).
    """
    layers = []
    d = in_features
    for _ in range(depth):
        layers += [nn.Linear(d, width, device=device), nn.GELU(), nn.LayerNorm([width], device=device)]
        d = width
    layers.append(nn.Linear(d, num_classes, device=device))
    return nn.Sequential(*layers)


def mnist_classifier(device=None) -> nn.Sequential:
    """Linear(784,256) - ReLU - LayerNorm(256) - Linear(256,10) - LogSoftmax."""
    return nn.Sequential(nn.Linear(784, 256, device=device), nn.ReLU(), nn.LayerNorm([256], device=device),
                         nn.Linear(256, 10, device=device), nn.LogSoftmax(-1))


class EmbeddingClassifier(nn.Module):
    """Mean-pooled Embedding(vocab, dim) -> Linear(dim, hidden) - SiLU - Dropout(p) - Linear(hidden, classes)."""

    def __init__(self, vocab: int = 50000, dim: int = 1024, hidden: int = 4096, num_classes: int = 512,
                 p_drop: float = 0.1, device=None):
        super().__init__()
        self.embed = nn.MeanPoolEmbedding(vocab, dim, device=device)
        self.head = nn.Sequential(nn.Linear(dim, hidden, device=device), nn.SiLU(), nn.Dropout(p_drop),
                                  nn.Linear(hidden, num_classes, device=device))

    @nn.tensor_io
    def forward(self, idx):
        return self.head(self.embed(idx))
