"""Runtime helpers, profiler, metrics."""
from . import profiler, runtime
from .graph import GraphedStep
from .profiler import StepTimer, profile

__all__ = ["runtime", "profiler", "profile", "StepTimer", "GraphedStep"]
