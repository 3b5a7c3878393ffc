"""``from ferrum_b200.prelude import *`` — the names of ``ferrum::prelude`` (ferrum/src/lib.rs:84-134)."""
from .autograd import GradientTape, NoGradGuard, backward, no_grad
from .core import DType, Device, FerrumError, Shape, Tensor
from .data import (DataLoader, Dataset, DistributedSampler, RandomSampler, SequentialSampler, Subset, TensorDataset,
                   train_test_split)
from .nn import (ELU, GELU, BatchNorm1d, Dropout, Embedding, LayerNorm, LeakyReLU, Linear, LogSoftmax, Module, ReLU,
                 Sequential, Sigmoid, SiLU, Softmax, Tanh, bce_loss, cross_entropy_loss, l1_loss, log_softmax,
                 mse_loss, nll_loss, smooth_l1_loss, softmax)
from .optim import (SGD, Adam, AdamConfig, CosineAnnealingLR, CosineAnnealingWarmRestarts, ExponentialLR,
                    LinearWarmupLR, LRScheduler, MultiStepLR, OneCycleLR, Optimizer, PlateauMode, ReduceLROnPlateau,
                    SGDConfig, StepLR)
from .parallel import (Backend, DistributedDataParallel, ProcessGroup, ReduceOp, barrier, get_rank, get_world_size,
                       init_process_group, is_main_process)
from .serialize import load, save

AutogradTensor = Tensor  # backward() is a method of Tensor
Result = object

__all__ = [n for n in dir() if not n.startswith("_")]
