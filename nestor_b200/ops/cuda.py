"""Kernel-backed op bodies (filled in by the modules under ``nestor_b200/ops/kernels``)."""
