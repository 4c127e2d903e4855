"""Operators: sm_100a kernels on CUDA tensors, PyTorch reference formulas on CPU tensors."""
from . import functional, native, reference  # noqa: F401
