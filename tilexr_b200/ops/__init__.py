"""Tensor-level operators backed by the native kernels."""
from . import collectives, ep, quant

__all__ = ["collectives", "ep", "quant"]
