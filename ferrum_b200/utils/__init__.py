"""Runtime helpers, profiler, metrics."""
from . import profiler, runtime
from .profiler import StepTimer, profile

__all__ = ["runtime", "profiler", "profile", "StepTimer"]
