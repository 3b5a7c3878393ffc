"""Index samplers (ferrum-data/src/sampler.rs:6-358).  Index generation runs in the native
host library (``csrc/host/sampler.cpp``: PCG32 + Fisher-Yates), seeded so that runs repeat."""
from __future__ import annotations

import ctypes
import itertools

import numpy as np

from .. import _lib

_auto_seed = itertools.count(0x5EED)


def _perm(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.int64)
    if n:
        _lib.host().fb_sampler_permutation(n, seed & 0xFFFFFFFFFFFFFFFF, out.ctypes.data)
    return out


class Sampler:
    """``len`` / ``is_empty`` / ``next_index`` plus Python iteration."""

    def __init__(self, indices):
        self.indices = np.asarray(indices, dtype=np.int64)
        self.current = 0

    def len(self) -> int:
        return len(self.indices)

    __len__ = len

    def is_empty(self) -> bool:
        return self.len() == 0

    def next_index(self):
        if self.current < len(self.indices):
            i = int(self.indices[self.current])
            self.current += 1
            return i
        return None

    def reset(self) -> None:
        self.current = 0

    def remaining(self) -> np.ndarray:
        """All indices not handed out yet (and marks them consumed)."""
        r = self.indices[self.current:]
        self.current = len(self.indices)
        return r

    def __iter__(self):
        return self

    def __next__(self):
        i = self.next_index()
        if i is None:
            raise StopIteration
        return i


class SequentialSampler(Sampler):
    def __init__(self, length: int):
        super().__init__(np.arange(length, dtype=np.int64))


class RandomSampler(Sampler):
    def __init__(self, length: int, seed: int | None = None):
        self.seed = next(_auto_seed) if seed is None else int(seed)
        self._epoch = 0
        super().__init__(_perm(length, self.seed))

    @classmethod
    def new(cls, length):
        return cls(length)

    @classmethod
    def with_seed(cls, length: int, seed: int):
        return cls(length, seed)

    def reshuffle(self) -> None:
        self._epoch += 1
        self.indices = _perm(len(self.indices), self.seed + 0x9E3779B97F4A7C15 * self._epoch)
        self.current = 0


class WeightedRandomSampler(Sampler):
    """``num_samples`` draws with replacement, probability proportional to ``weights``."""

    def __init__(self, weights, num_samples: int, seed: int | None = None):
        w = np.ascontiguousarray(weights, dtype=np.float64)
        out = np.empty(num_samples, dtype=np.int64)
        seed = next(_auto_seed) if seed is None else int(seed)
        rc = _lib.host().fb_sampler_weighted(w.ctypes.data, len(w), num_samples, seed, out.ctypes.data)
        if rc != 0:
            raise ValueError("weights must be non-negative with a positive sum")
        self.weights = w
        super().__init__(out)


class SubsetRandomSampler(Sampler):
    def __init__(self, indices, seed: int | None = None):
        src = np.ascontiguousarray(indices, dtype=np.int64)
        out = np.empty_like(src)
        seed = next(_auto_seed) if seed is None else int(seed)
        if len(src):
            _lib.host().fb_sampler_subset(src.ctypes.data, len(src), seed, out.ctypes.data)
        super().__init__(out)


class DistributedSampler(Sampler):
    """This rank's share of the dataset: the index list is padded by wrap-around to a multiple of
    ``num_replicas``, shuffled with a seed common to all ranks, and cut into contiguous rank slices."""

    def __init__(self, length: int, num_replicas: int, rank: int, shuffle: bool = True, seed: int = 0):
        if not 0 <= rank < num_replicas:
            raise ValueError(f"rank {rank} out of range for {num_replicas} replicas")
        self.length, self.num_replicas, self.rank, self.shuffle, self.seed = length, num_replicas, rank, shuffle, seed
        super().__init__(self._generate(seed))

    def _generate(self, seed: int) -> np.ndarray:
        per = -(-self.length // self.num_replicas)
        out = np.empty(per, dtype=np.int64)
        n = _lib.host().fb_sampler_distributed(self.length, self.num_replicas, self.rank, 1 if self.shuffle else 0,
                                               seed & 0xFFFFFFFFFFFFFFFF, out.ctypes.data, per)
        if n < 0:
            raise ValueError("invalid distributed sampler configuration")
        return out[:n]

    def set_epoch(self, epoch: int) -> None:
        self.indices = self._generate(self.seed + int(epoch))
        self.current = 0


class BatchSampler:
    """Groups a sampler's indices into lists of ``batch_size`` (sampler.rs:193-240)."""

    def __init__(self, sampler: Sampler, batch_size: int, drop_last: bool = False):
        if batch_size <= 0:
            raise ValueError("batch_size must be positive")
        self.sampler, self.batch_size, self.drop_last = sampler, int(batch_size), bool(drop_last)

    def len(self) -> int:
        return int(_lib.host().fb_sampler_num_batches(self.sampler.len(), self.batch_size,
                                                      1 if self.drop_last else 0))

    __len__ = len

    def __iter__(self):
        return self

    def next_batch(self):
        """The next batch as an int64 array, or None when exhausted."""
        s = self.sampler
        lo = s.current
        hi = min(lo + self.batch_size, len(s.indices))
        if hi <= lo or (self.drop_last and hi - lo < self.batch_size):
            s.current = len(s.indices)
            return None
        s.current = hi
        return s.indices[lo:hi]

    def __next__(self):
        b = self.next_batch()
        if b is None:
            raise StopIteration
        return b.tolist()


def zipf_indices(vocab: int, s: float, n: int, seed: int = 0) -> np.ndarray:
    """``n`` token ids ~ Zipf(s) over ``[0, vocab)`` (synthetic text for the embedding benchmark)."""
    out = np.empty(n, dtype=np.int64)
    if _lib.host().fb_sampler_zipf(vocab, float(s), n, seed, out.ctypes.data) != 0:
        raise ValueError("vocab must be positive")
    return out
