"""Runtime helpers, profiler, logging."""
