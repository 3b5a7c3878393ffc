"""Datasets (ferrum-data/src/dataset.rs:8-200)."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..core import Tensor, _unwrap
from .sampler import _perm


class Dataset:
    """``len`` / ``is_empty`` / ``get(i)``; also indexable and iterable."""

    def len(self) -> int:
        raise NotImplementedError

    def get(self, index: int):
        raise NotImplementedError

    def is_empty(self) -> bool:
        return self.len() == 0

    def __len__(self):
        return self.len()

    def __getitem__(self, i):
        if i < 0:
            i += self.len()
        if not 0 <= i < self.len():
            raise IndexError(i)
        return self.get(i)


class TensorDataset(Dataset):
    """Pairs of (input, target).

    ``TensorDataset(inputs, targets)`` with two *lists* stores one entry per sample, as the
    reference does (dataset.rs:34-41).  ``TensorDataset.from_tensors(x, y)`` keeps the two
    stacked tensors and yields one sample per row of dim 0 — what the reference's docstring
    promises (its code stores a single sample); such a dataset can live on the GPU, where
    ``DataLoader`` fetches a whole batch with one row-gather kernel.
    """

    def __init__(self, inputs, targets):
        if isinstance(inputs, (Tensor, torch.Tensor)) and isinstance(targets, (Tensor, torch.Tensor)):
            self.stacked = True
            self.inputs, self.targets = _unwrap(inputs), _unwrap(targets)
            if self.inputs.shape[0] != self.targets.shape[0]:
                raise ValueError("Inputs and targets must have the same length")
        else:
            self.stacked = False
            self.inputs, self.targets = list(inputs), list(targets)
            if len(self.inputs) != len(self.targets):
                raise ValueError("Inputs and targets must have the same length")

    @classmethod
    def new(cls, inputs, targets):
        return cls(inputs, targets)

    @classmethod
    def from_tensors(cls, inputs, targets):
        return cls(inputs, targets)

    def len(self) -> int:
        return self.inputs.shape[0] if self.stacked else len(self.inputs)

    def get(self, index: int):
        if self.stacked:
            return Tensor(self.inputs[index]), Tensor(self.targets[index])
        return self.inputs[index], self.targets[index]

    def get_batch(self, indices):
        """Rows ``indices`` of both tensors as two stacked tensors (device row-gather on CUDA)."""
        if not self.stacked:
            raise TypeError("get_batch needs a dataset built from stacked tensors")
        from ..ops import functional as F

        idx = torch.as_tensor(np.asarray(indices, dtype=np.int64))
        if self.inputs.is_cuda:
            idx = idx.to(self.inputs.device, non_blocking=True)
        return Tensor(F.gather_rows(self.inputs, idx)), Tensor(F.gather_rows(self.targets, idx))


class MapDataset(Dataset):
    def __init__(self, dataset: Dataset, transform):
        self.dataset, self.transform = dataset, transform

    def len(self):
        return self.dataset.len()

    def get(self, index):
        return self.transform(self.dataset.get(index))


class ConcatDataset(Dataset):
    def __init__(self, datasets):
        self.datasets = list(datasets)
        self.cumulative = np.cumsum([d.len() for d in self.datasets]).tolist()

    def len(self):
        return self.cumulative[-1] if self.cumulative else 0

    def get(self, index):
        for k, end in enumerate(self.cumulative):
            if index < end:
                start = self.cumulative[k - 1] if k else 0
                return self.datasets[k].get(index - start)
        raise IndexError(index)


class Subset(Dataset):
    def __init__(self, dataset: Dataset, indices):
        self.dataset, self.indices = dataset, [int(i) for i in indices]

    def len(self):
        return len(self.indices)

    def get(self, index):
        return self.dataset.get(self.indices[index])


def train_test_split(dataset: Dataset, test_ratio: float, shuffle: bool = True, seed: int = 0):
    """(train, test) subsets; the test part has ``ceil(n * test_ratio)`` samples (dataset.rs:173-200)."""
    n = dataset.len()
    test_size = int(math.ceil(n * test_ratio))
    train_size = n - test_size
    idx = _perm(n, seed).tolist() if shuffle else list(range(n))
    return Subset(dataset, idx[:train_size]), Subset(dataset, idx[train_size:])
