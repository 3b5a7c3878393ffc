"""Distributed training (ferrum-distributed): process groups, collectives over NVLink, DistributedDataParallel."""
from .backend import (AlreadyInitialized, Backend, BackendConfig, CommunicationError, DistributedError,
                      InternalError, InvalidConfiguration, InvalidRank, NotInitialized, ReduceOp, TensorError, Timeout,
                      UnsupportedBackend)
from .ddp import DistributedDataParallel, GradientBucket, GradientHook
from .process_group import (ProcessGroup, barrier, destroy_process_group, get_rank, get_world, get_world_size,
                            init_process_group, init_process_group_from_env, is_initialized, is_main_process,
                            leave_process_group, new_group)
from .symm import SymmetricArena

Collectives = ProcessGroup  # the trait's eight operations are methods of the group

__all__ = [
    "Backend", "BackendConfig", "ReduceOp", "ProcessGroup", "Collectives", "new_group", "init_process_group",
    "init_process_group_from_env", "get_world", "is_initialized", "destroy_process_group", "leave_process_group",
    "get_rank",
    "get_world_size", "is_main_process", "barrier", "DistributedDataParallel", "GradientBucket", "GradientHook",
    "SymmetricArena", "DistributedError", "AlreadyInitialized", "NotInitialized", "InvalidRank",
    "CommunicationError", "Timeout", "UnsupportedBackend", "InvalidConfiguration", "TensorError",
    "InternalError",
]
