"""Runtime helpers, profiler, metrics."""
from . import profiler, runtime
from .graph import GraphedStep, HostReadback
from .profiler import StepTimer, profile

__all__ = ["runtime", "profiler", "profile", "StepTimer", "GraphedStep", "HostReadback"]
