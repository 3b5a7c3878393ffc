"""The eight learning-rate schedulers of ferrum-optim/src/scheduler.rs:8-542.

They are closed-form functions of a step counter and do not hold an optimizer:
the training loop calls ``optimizer.set_learning_rate(scheduler.get_lr())``.
``attach(optimizer)`` is a convenience that makes ``step()`` push the new rate.
"""
from __future__ import annotations

import enum
import math


class LRScheduler:
    """``get_lr`` / ``step`` / ``current_step`` / ``reset`` (scheduler.rs:8-21)."""

    _optimizer = None

    def get_lr(self) -> float:
        raise NotImplementedError

    def _advance(self) -> None:
        raise NotImplementedError

    def step(self) -> None:
        self._advance()
        if self._optimizer is not None:
            self._optimizer.set_learning_rate(self.get_lr())

    def current_step(self) -> int:
        raise NotImplementedError

    def reset(self) -> None:
        raise NotImplementedError

    def attach(self, optimizer) -> "LRScheduler":
        self._optimizer = optimizer
        optimizer.set_learning_rate(self.get_lr())
        return self

    def state_dict(self) -> dict:
        return {k: v for k, v in self.__dict__.items() if not k.startswith("_")}

    def load_state_dict(self, sd: dict) -> None:
        self.__dict__.update(sd)


class _EpochScheduler(LRScheduler):
    def __init__(self):
        self.current_epoch = 0

    def _advance(self):
        self.current_epoch += 1

    def current_step(self):
        return self.current_epoch

    def reset(self):
        self.current_epoch = 0


class StepLR(_EpochScheduler):
    def __init__(self, base_lr: float, step_size: int, gamma: float):
        super().__init__()
        self.base_lr, self.step_size, self.gamma = float(base_lr), int(step_size), float(gamma)

    def get_lr(self):
        return self.base_lr * self.gamma ** (self.current_epoch // self.step_size)


class MultiStepLR(_EpochScheduler):
    def __init__(self, base_lr: float, milestones, gamma: float):
        super().__init__()
        self.base_lr, self.milestones, self.gamma = float(base_lr), sorted(int(m) for m in milestones), float(gamma)

    def get_lr(self):
        return self.base_lr * self.gamma ** sum(1 for m in self.milestones if m <= self.current_epoch)


class ExponentialLR(_EpochScheduler):
    def __init__(self, base_lr: float, gamma: float):
        super().__init__()
        self.base_lr, self.gamma = float(base_lr), float(gamma)

    def get_lr(self):
        return self.base_lr * self.gamma ** self.current_epoch


class CosineAnnealingLR(_EpochScheduler):
    def __init__(self, base_lr: float, t_max: int, eta_min: float = 0.0):
        super().__init__()
        self.base_lr, self.t_max, self.eta_min = float(base_lr), int(t_max), float(eta_min)

    def get_lr(self):
        t = min(self.current_epoch, self.t_max)
        return self.eta_min + 0.5 * (self.base_lr - self.eta_min) * (1.0 + math.cos(math.pi * t / self.t_max))


class CosineAnnealingWarmRestarts(LRScheduler):
    def __init__(self, base_lr: float, t_0: int, t_mult: int = 1, eta_min: float = 0.0):
        self.base_lr, self.t_0, self.t_mult, self.eta_min = float(base_lr), int(t_0), int(t_mult), float(eta_min)
        self.current_epoch, self.current_cycle, self.current_t_i = 0, 0, int(t_0)

    def get_lr(self):
        t_cur = self.current_epoch % self.current_t_i
        return self.eta_min + 0.5 * (self.base_lr - self.eta_min) * (
            1.0 + math.cos(math.pi * t_cur / self.current_t_i))

    def _advance(self):
        self.current_epoch += 1
        if self.current_epoch >= self.current_t_i:
            self.current_epoch = 0
            self.current_cycle += 1
            if self.t_mult > 1:
                self.current_t_i *= self.t_mult

    def current_step(self):
        return self.current_epoch + self.current_cycle * self.t_0

    def reset(self):
        self.current_epoch, self.current_cycle, self.current_t_i = 0, 0, self.t_0


class LinearWarmupLR(LRScheduler):
    def __init__(self, base_lr: float, warmup_steps: int, total_steps: int):
        self.base_lr, self.warmup_steps, self.total_steps = float(base_lr), int(warmup_steps), int(total_steps)
        self.step_count = 0

    def get_lr(self):
        if self.step_count < self.warmup_steps:
            return self.base_lr * (self.step_count / self.warmup_steps)
        remaining = max(self.total_steps - self.step_count, 0)
        decay = self.total_steps - self.warmup_steps
        return self.base_lr * max(remaining / decay, 0.0) if decay > 0 else 0.0

    def _advance(self):
        self.step_count += 1

    def current_step(self):
        return self.step_count

    def reset(self):
        self.step_count = 0


class OneCycleLR(LRScheduler):
    def __init__(self, max_lr: float, total_steps: int, pct_start: float = 0.3, div_factor: float = 25.0,
                 final_div_factor: float = 1e4):
        self.max_lr, self.total_steps = float(max_lr), int(total_steps)
        self.pct_start, self.div_factor, self.final_div_factor = float(pct_start), float(div_factor), float(
            final_div_factor)
        self.step_count = 0

    @classmethod
    def new_default(cls, max_lr: float, total_steps: int):
        return cls(max_lr, total_steps)

    def get_lr(self):
        initial = self.max_lr / self.div_factor
        final = initial / self.final_div_factor
        up = int(self.total_steps * self.pct_start)
        if self.step_count < up:
            return initial + (self.max_lr - initial) * (self.step_count / up)
        down = (self.step_count - up) / max(self.total_steps - up, 1)
        return final + (self.max_lr - final) * (1.0 + math.cos(math.pi * down)) / 2.0

    def _advance(self):
        self.step_count = min(self.step_count + 1, self.total_steps)

    def current_step(self):
        return self.step_count

    def reset(self):
        self.step_count = 0


class PlateauMode(enum.Enum):
    Min = "min"
    Max = "max"


class ReduceLROnPlateau(LRScheduler):
    def __init__(self, base_lr: float, mode: PlateauMode = PlateauMode.Min, factor: float = 0.1, patience: int = 10,
                 min_lr: float = 0.0):
        self.base_lr = self.current_lr = float(base_lr)
        self.mode, self.factor, self.patience, self.min_lr = mode, float(factor), int(patience), float(min_lr)
        self.threshold = 1e-4
        self.best = math.inf if mode == PlateauMode.Min else -math.inf
        self.num_bad_epochs = 0
        self.current_epoch = 0

    def step_with_metric(self, metric: float) -> None:
        self.current_epoch += 1
        if self.mode == PlateauMode.Min:
            better = metric < self.best * (1.0 - self.threshold)
        else:
            better = metric > self.best * (1.0 + self.threshold)
        if better:
            self.best, self.num_bad_epochs = metric, 0
        else:
            self.num_bad_epochs += 1
            if self.num_bad_epochs >= self.patience:
                self.current_lr = max(self.current_lr * self.factor, self.min_lr)
                self.num_bad_epochs = 0
        if self._optimizer is not None:
            self._optimizer.set_learning_rate(self.get_lr())

    def get_lr(self):
        return self.current_lr

    def _advance(self):
        self.current_epoch += 1

    def current_step(self):
        return self.current_epoch

    def reset(self):
        self.current_lr = self.base_lr
        self.best = math.inf if self.mode == PlateauMode.Min else -math.inf
        self.num_bad_epochs = 0
        self.current_epoch = 0
