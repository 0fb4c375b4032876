"""Kernel-level operators. `ops` carries the grouped GEMM, the weight gradient and the row gather with the
reference's names (scattermoe/kernels/ops.py); `single` (imported on demand, as in the reference) the decode matvec."""
from . import ops

__all__ = ["ops"]
