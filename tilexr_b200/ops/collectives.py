"""Collectives on torch tensors (current CUDA stream).

Each function issues kernels and returns without synchronising, like the C API
(csrc/include/tilexr_collectives.h).  Output tensors that live in registered memory
(``Comm.symm_empty`` / ``Comm.register``) are written by the peers directly.

CPU tensors on a host-memory communicator (``init_from_torch_distributed(host_memory=True)``, the no-GPU plumbing
mode) take the host kernels instead: the same windows, flags and launch epochs, blocking, sums in fp32 only.
"""
from __future__ import annotations

import enum
from typing import Optional

import torch

from .. import _C


class ReduceOp(enum.IntEnum):
    SUM = 0
    PROD = 1
    MAX = 2
    MIN = 3


HOST_TILE_BYTES = 16384


def _host_sum_only(x: torch.Tensor, op) -> None:
    if int(op) != int(ReduceOp.SUM) or x.dtype != torch.float32:
        raise ValueError("host-memory communicators reduce fp32 sums only")


def _into(out: Optional[torch.Tensor], value: torch.Tensor) -> torch.Tensor:
    if out is None:
        return value
    out.copy_(value.view_as(out))
    return out


def all_gather(comm, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    x = x.contiguous()
    if not x.is_cuda:
        if out is None:
            out = torch.empty((comm.world_size,) + tuple(x.shape), dtype=x.dtype)
        _C.host_all_gather(comm, x, out, HOST_TILE_BYTES)
        return out
    if out is None:
        out = torch.empty((comm.world_size,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    _C.all_gather(comm, x, out)
    return out


def all_to_all(comm, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Equal split along dim 0: chunk p of ``x`` goes to rank p."""
    x = x.contiguous()
    if not x.is_cuda:
        return _into(out, _C.host_all_to_all(comm, x, HOST_TILE_BYTES))
    if out is None:
        out = torch.empty_like(x)
    _C.all_to_all(comm, x, out)
    return out


def all_reduce(comm, x: torch.Tensor, op: ReduceOp = ReduceOp.SUM, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    x = x.contiguous()
    if not x.is_cuda:
        _host_sum_only(x, op)
        return _into(out, _C.host_all_reduce(comm, x.reshape(-1)).view_as(x))
    if out is None:
        out = torch.empty_like(x)
    _C.all_reduce(comm, x, out, int(op))
    return out


def reduce_scatter(comm, x: torch.Tensor, op: ReduceOp = ReduceOp.SUM, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x`` holds world_size equal chunks along dim 0; returns the reduction of chunk ``rank``."""
    x = x.contiguous()
    if not x.is_cuda:
        _host_sum_only(x, op)
        shape = list(x.shape)
        shape[0] //= comm.world_size
        return _into(out, _C.host_reduce_scatter(comm, x.reshape(-1)).view(shape))
    if out is None:
        shape = list(x.shape)
        shape[0] //= comm.world_size
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    _C.reduce_scatter(comm, x, out, int(op))
    return out


def broadcast(comm, x: torch.Tensor, root: int = 0) -> torch.Tensor:
    if not x.is_cuda:
        if not x.is_contiguous():
            raise ValueError("broadcast works in place on a contiguous tensor")
        _C.host_broadcast(comm, x, root, HOST_TILE_BYTES)
        return x
    _C.broadcast(comm, x, root)
    return x


def profile_probe(comm, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty_like(x)
    _C.profile_probe(comm, x.contiguous(), out)
    return out


AR_AUTO, AR_ONE_SHOT, AR_TWO_SHOT = 0, 1, 2


def all_reduce_rmsnorm(comm, x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6,
                       residual: Optional[torch.Tensor] = None, algo: int = AR_AUTO,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = RMSNorm(all_reduce(x) + residual) * gamma`` in one kernel; ``residual`` is updated in
    place with the pre-norm sum.  ``algo`` forces one-shot or two-shot (default: by size)."""
    return _C.all_reduce_rmsnorm(comm, x.contiguous(), residual, gamma, eps, algo, out)


def all_reduce_quant(comm, x: torch.Tensor, scale: torch.Tensor, offset: float = 0.0) -> torch.Tensor:
    """Sum over ranks of ``(x + offset) * scale`` for int8 ``x``; ``scale`` (fp16 / bf16, one element or one per
    channel of the last dimension) gives the output dtype.  int8 crosses NVLink in the first hop, sums are fp32."""
    return _C.all_reduce_quant(comm, x.contiguous(), scale.contiguous(), float(offset))


def all_to_all_transpose(comm, x: torch.Tensor) -> torch.Tensor:
    """``x`` is [rows, width]; returns [world, rows, width // world] where entry ``s`` is column block ``rank`` of rank
    ``s``'s matrix: the sequence-parallel <-> head-parallel exchange, with the transpose done by the sending kernel."""
    return _C.all_to_all_transpose(comm, x.contiguous())
