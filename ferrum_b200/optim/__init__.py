"""Optimizers, LR schedulers and mixed-precision helpers (ferrum-optim)."""
from .amp import (Autocast, GradScaler, clip_grad_norm, clip_grad_value, has_inf_or_nan, to_bfloat16, to_float,
                  to_half)
from .optimizers import SGD, Adam, AdamConfig, Optimizer, SGDConfig
from .scheduler import (CosineAnnealingLR, CosineAnnealingWarmRestarts, ExponentialLR, LinearWarmupLR, LRScheduler,
                        MultiStepLR, OneCycleLR, PlateauMode, ReduceLROnPlateau, StepLR)

__all__ = [
    "Optimizer", "SGD", "SGDConfig", "Adam", "AdamConfig", "LRScheduler", "StepLR", "MultiStepLR", "ExponentialLR",
    "CosineAnnealingLR", "CosineAnnealingWarmRestarts", "LinearWarmupLR", "OneCycleLR", "ReduceLROnPlateau",
    "PlateauMode", "GradScaler", "Autocast", "to_half", "to_bfloat16", "to_float", "has_inf_or_nan",
    "clip_grad_norm", "clip_grad_value",
]
