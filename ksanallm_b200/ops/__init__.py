"""Operator layer: hand-written sm_100a kernels (``native``) for CUDA tensors and plain PyTorch
statements (``reference``) for CPU tensors and as test oracles."""
from . import reference  # noqa: F401
from . import native  # noqa: F401
