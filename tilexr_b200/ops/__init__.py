"""Tensor-level operators backed by the native kernels."""
from . import collectives, ep, gemm, quant

__all__ = ["collectives", "ep", "gemm", "quant"]
