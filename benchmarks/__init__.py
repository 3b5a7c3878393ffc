"""Measurement tools (GEMM / kernel / collective sweeps); run as ``python -m benchmarks.<name>`` from the repository root."""
