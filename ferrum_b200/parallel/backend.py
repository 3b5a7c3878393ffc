"""Backends, configuration, reduce operations and errors of the distributed layer
(ferrum-distributed/src/{backend,collectives,error}.rs)."""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass, replace

import torch

from ..core import FerrumError


class DistributedError(FerrumError):
    pass


class AlreadyInitialized(DistributedError):
    def __init__(self):
        super().__init__("Process group already initialized")


class NotInitialized(DistributedError):
    def __init__(self):
        super().__init__("Process group not initialized")


class InvalidRank(DistributedError):
    def __init__(self, rank, world):
        super().__init__(f"Invalid rank {rank} for world size {world}")


class CommunicationError(DistributedError):
    def __init__(self, msg):
        super().__init__(f"Communication error: {msg}")


class Timeout(DistributedError):
    def __init__(self, what):
        super().__init__(f"Timeout during {what}")


class UnsupportedBackend(DistributedError):
    def __init__(self, name):
        super().__init__(f"Backend not supported: {name}")


class InvalidConfiguration(DistributedError):
    def __init__(self, msg):
        super().__init__(f"Invalid configuration: {msg}")


class TensorError(DistributedError):
    def __init__(self, msg):
        super().__init__(f"Tensor error: {msg}")


class InternalError(DistributedError):
    """``DistributedError::InternalError`` (ferrum-distributed/src/error.rs:40-42)."""

    def __init__(self, msg):
        super().__init__(f"Internal error: {msg}")


class Backend(enum.Enum):
    """``Nvlink`` is this package's own transport (sm_100a kernels over peer memory); ``Nccl`` is the library
    baseline; ``Gloo`` runs CPU ranks; ``Mpi`` is declared by the reference and not provided."""

    Nccl = "nccl"
    Gloo = "gloo"
    Mpi = "mpi"
    Nvlink = "nvlink"

    def is_available(self) -> bool:
        if self is Backend.Gloo:
            return torch.distributed.is_available() and torch.distributed.is_gloo_available()
        if self is Backend.Nccl:
            return torch.cuda.is_available() and torch.distributed.is_nccl_available()
        if self is Backend.Nvlink:
            return torch.cuda.is_available()
        return False

    def name_str(self) -> str:
        return self.value

    def __str__(self):
        return self.value

    @staticmethod
    def from_str(s: str) -> "Backend":
        try:
            return Backend(s.strip().lower())
        except ValueError:
            raise UnsupportedBackend(s) from None


@dataclass
class BackendConfig:
    master_addr: str = "127.0.0.1"
    master_port: int = 29500
    timeout_seconds: int = 1800
    num_threads: int = 4

    @classmethod
    def from_env(cls) -> "BackendConfig":
        c = cls()
        if os.environ.get("MASTER_ADDR"):
            c.master_addr = os.environ["MASTER_ADDR"]
        if os.environ.get("MASTER_PORT"):
            c.master_port = int(os.environ["MASTER_PORT"])
        if os.environ.get("DIST_TIMEOUT"):
            c.timeout_seconds = int(os.environ["DIST_TIMEOUT"])
        return c

    def with_master_addr(self, addr: str) -> "BackendConfig":
        return replace(self, master_addr=addr)

    def with_master_port(self, port: int) -> "BackendConfig":
        return replace(self, master_port=int(port))

    def with_timeout(self, seconds: int) -> "BackendConfig":
        return replace(self, timeout_seconds=int(seconds))

    def device_wait_ns(self) -> int:
        """Bound of a single device-side wait: the configured timeout, capped (default 10 s,
        ``FERRUM_DEVICE_WAIT_S``) so that a lost peer cannot keep a shared GPU spinning for long."""
        cap = float(os.environ.get("FERRUM_DEVICE_WAIT_S", "10"))
        return int(min(float(self.timeout_seconds), cap) * 1e9)


class ReduceOp(enum.Enum):
    Sum = 0
    Product = 1
    Min = 2
    Max = 3
    Average = 4

    def apply(self, a: float, b: float) -> float:
        """Pairwise combination (collectives.rs:18-32); ``Average`` sums here, the division happens at the end."""
        if self is ReduceOp.Product:
            return a * b
        if self is ReduceOp.Min:
            return min(a, b)
        if self is ReduceOp.Max:
            return max(a, b)
        return a + b
