"""Model zoo (ferrum-nn/src/models.rs) and the benchmark networks."""
from .mlp import MLP, EmbeddingClassifier, mnist_classifier, wide_mlp
from .vision import VGG, BasicBlock, ResNet

__all__ = ["MLP", "wide_mlp", "mnist_classifier", "EmbeddingClassifier", "BasicBlock", "ResNet", "VGG"]
