"""tcgen05 GEMM and its fusions with collectives (csrc/include/tilexr_fused.h).

Weights follow the ``torch.nn.Linear`` convention: ``b`` is ``[N, K]`` and the product is
``a @ b.T``.
"""
from __future__ import annotations

import torch

from .. import _C


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a[M,K] @ b[N,K].T`` on the tensor cores (fp16 / bf16, fp32 accumulation)."""
    return _C.matmul(a.contiguous(), b.contiguous())


def matmul_fp8(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``alpha * a @ b.T`` for fp8 operands (both float8_e4m3fn or both float8_e5m2; a [M, K], b [N, K], K % 16 == 0) with fp32
    accumulation on the 8-bit tensor-core path; ``alpha`` is the product of the two per-tensor dequantisation scales."""
    return _C.matmul_fp8(a.contiguous(), b.contiguous(), float(alpha), out_dtype)


def all_gather_matmul(comm, a_shard: torch.Tensor, b: torch.Tensor, staging: torch.Tensor) -> torch.Tensor:
    """``all_gather(a_shard) @ b.T`` with the gather overlapped tile by tile.

    ``staging`` is a ``comm.symm_empty([world * rows, K], dtype)`` buffer reused across calls.
    """
    return _C.all_gather_matmul(comm, a_shard.contiguous(), staging, b.contiguous())


def matmul_reduce_scatter(comm, a: torch.Tensor, b: torch.Tensor, staging: torch.Tensor) -> torch.Tensor:
    """``reduce_scatter(a @ b.T)`` along rows; ``staging`` is ``comm.symm_empty([M, N], dtype)``."""
    return _C.matmul_reduce_scatter(comm, a.contiguous(), b.contiguous(), staging)
