"""Datasets, samplers, loaders and transforms (ferrum-data)."""
from .dataloader import CollatedDataLoader, DataLoader, DevicePrefetcher, default_collate
from .dataset import ConcatDataset, Dataset, MapDataset, Subset, TensorDataset, train_test_split
from .sampler import (BatchSampler, DistributedSampler, RandomSampler, Sampler, SequentialSampler,
                      SubsetRandomSampler, WeightedRandomSampler, zipf_indices)
from .transform import Compose, GaussianNoise, Identity, Lambda, Normalize, Scale, ToOneHot, Transform

__all__ = [
    "Dataset", "TensorDataset", "MapDataset", "ConcatDataset", "Subset", "train_test_split", "DataLoader",
    "CollatedDataLoader", "DevicePrefetcher", "default_collate", "Sampler", "SequentialSampler", "RandomSampler",
    "WeightedRandomSampler", "BatchSampler", "SubsetRandomSampler", "DistributedSampler", "zipf_indices",
    "Transform", "Compose", "Normalize", "Scale", "GaussianNoise", "Identity", "ToOneHot", "Lambda",
]
