"""Collectives through the NVSwitch multicast object (NVLS), C API ``TileXRNvls*`` in
``csrc/include/tilexr_collectives.h``, kernels in ``csrc/collectives/nvls_kernels.cu``.

``multimem`` loads reduce inside the switch and ``multimem`` stores reach every rank's copy of a
buffer, so an all-reduce moves 2/R of the message out of each GPU instead of (R-1) x (one-shot
pushes) or 2 (R-1)/R x (two-shot).  The buffer has to be a symmetric allocation bound to a
multicast object.  The communicator allocates it (CUDA virtual-memory API, POSIX descriptors traded
over the library's own exchange, one multicast object per allocation: csrc/comm/vmm.cpp), and the same
mechanism backs the communicator's window, so ``txr.all_reduce`` and friends take the in-switch path
by themselves for large messages.  The kernels synchronise the ranks through the communicator's flag
windows with bounded waits.

    ws = nvls.Workspace(comm, 64 << 20)              # collective: every rank of the group calls it
    buf = ws.view(torch.bfloat16, n)                  # a tensor inside this rank's copy
    buf.copy_(x); ws.all_reduce_(buf)                 # in place, every rank gets the same bits
    y = ws.all_reduce(x)                              # convenience: copy in, reduce, copy out

The reference has no in-fabric reduction; its all-reduce variants (src/collectives/kernels/allreduce_*.h)
move every byte through the ranks' memories.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _C


class NvlsUnavailable(RuntimeError):
    """The GPUs of the group cannot be bound to one multicast object (no NVSwitch, or the driver refuses)."""


class Workspace:
    """A symmetric buffer of ``nbytes`` per rank, bound to one multicast object.

    ``group`` is the ``torch.distributed`` process group whose ranks are the communicator's ranks in
    the same order (default: the world group).  Creating a workspace is a collective call.
    """

    def __init__(self, comm, nbytes: int, group=None, device: Optional[torch.device] = None):
        nbytes = (int(nbytes) + 255) // 256 * 256
        self.comm = comm
        self.nbytes = nbytes
        self.handle = None
        if comm.nvls_available():
            # The communicator's own allocator: virtual-memory API, POSIX descriptors over the library's
            # exchange, every copy bound to one multicast object (csrc/comm/vmm.cpp).
            self.buffer = comm.symm_empty([nbytes], torch.uint8)
            self.mc_base = int(comm.multicast_ptr(self.buffer))
            self.local_base = self.buffer.data_ptr()
            if self.mc_base == 0:
                raise NvlsUnavailable("the allocation has no multicast address on this system")
            self.source = "runtime"
            return
        self._init_from_torch(nbytes, group, device)

    def _init_from_torch(self, nbytes: int, group, device) -> None:
        """Where the communicator has no multicast object of its own (created with TILEXR_ENABLE_VMM=0 or
        TILEXR_ENABLE_NVLS=0, say), a buffer of ``torch.distributed._symmetric_memory`` serves."""
        import torch.distributed as dist

        comm = self.comm
        if not dist.is_initialized():
            raise NvlsUnavailable("the communicator has no multicast object and torch.distributed is not initialised")
        import torch.distributed._symmetric_memory as symm

        group = group if group is not None else dist.group.WORLD
        if dist.get_world_size(group) != comm.world_size or dist.get_rank(group) != comm.rank:
            raise ValueError("the process group and the communicator must have the same ranks in the same order")
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        try:
            self.buffer = symm.empty(nbytes, dtype=torch.uint8, device=device)
            self.handle = symm.rendezvous(self.buffer, group)
        except RuntimeError as e:      # no symmetric-memory support on this system (driver, fabric, or permissions)
            raise NvlsUnavailable(str(e).splitlines()[0] if str(e) else "symmetric memory allocation failed") from e
        self.mc_base = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if self.mc_base == 0:
            raise NvlsUnavailable("the symmetric allocation has no multicast address on this system")
        # The multicast address maps the whole allocation; the tensor may start inside it.
        self.local_base = int(self.handle.buffer_ptrs[comm.rank])
        if not (self.local_base <= self.buffer.data_ptr() < self.local_base + max(int(self.handle.buffer_size), 1)):
            raise NvlsUnavailable("the symmetric tensor does not lie in the mapped allocation")
        self.source = "torch"

    # ---- views ------------------------------------------------------------------------------
    def view(self, dtype: torch.dtype, numel: int, offset_bytes: int = 0) -> torch.Tensor:
        """``numel`` elements of ``dtype`` at ``offset_bytes`` (a multiple of 16) of this rank's copy."""
        size = numel * torch.empty((), dtype=dtype).element_size()
        if offset_bytes % 16 != 0 or offset_bytes < 0 or offset_bytes + size > self.nbytes:
            raise ValueError(f"view of {size} bytes at offset {offset_bytes} does not fit the {self.nbytes}-byte workspace")
        return self.buffer[offset_bytes:offset_bytes + size].view(dtype)

    def _mc_addr(self, t: torch.Tensor) -> int:
        inside = t.data_ptr() - self.buffer.data_ptr()
        if inside < 0 or inside + t.numel() * t.element_size() > self.nbytes or not t.is_contiguous():
            raise ValueError("the tensor is not a contiguous view of this workspace")
        off = t.data_ptr() - self.local_base
        if off % 16 != 0 or (t.numel() * t.element_size()) % 16 != 0:
            raise ValueError("views start and end on 16-byte boundaries")
        return self.mc_base + off

    # ---- in-place operations on views -----------------------------------------------------------
    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        """Sum of every rank's ``t`` (same offset on all ranks), in place; bf16, fp16 or fp32."""
        _C.nvls_all_reduce(self.comm, self._mc_addr(t), t)
        return t

    def reduce_scatter(self, t: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``t`` holds world_size equal slices; returns the sum of slice ``rank`` (a local tensor)."""
        R = self.comm.world_size
        if out is None:
            out = torch.empty(t.numel() // R, dtype=t.dtype, device=t.device)
        _C.nvls_reduce_scatter(self.comm, self._mc_addr(t), t, out)
        return out

    def all_gather_(self, shard: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        """``shard`` (any local tensor) lands at slice ``rank`` of the view ``t`` on every rank."""
        _C.nvls_all_gather(self.comm, shard.contiguous(), self._mc_addr(t), t)
        return t

    def broadcast_(self, t: torch.Tensor, root: int, src: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The root's ``src`` (default: its own copy of the view) lands in the view ``t`` on every rank."""
        if self.comm.rank == root and src is None:
            src = t
        _C.nvls_broadcast(self.comm, src.contiguous() if src is not None else None, self._mc_addr(t), t, root)
        return t

    def all_reduce_rmsnorm_(self, x: torch.Tensor, gamma: torch.Tensor, residual: Optional[torch.Tensor] = None,
                            eps: float = 1e-6, y: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``y = RMSNorm(sum over ranks of x + residual) * gamma`` and ``residual <- sum + residual`` in one kernel.

        ``x`` [rows, h] (fp16 / bf16), ``y`` (default: ``x`` itself) and ``residual`` are views of the workspace at the
        same offsets on every rank; every rank holds the same residual and receives the same ``y`` and residual.
        A row's owner reduces it inside the switch, normalises it and multicasts the results.
        """
        if y is None:
            y = x
        _C.nvls_all_reduce_rmsnorm(self.comm, self._mc_addr(x), x, self._mc_addr(residual) if residual is not None else 0, residual,
                                   gamma.contiguous(), float(eps), self._mc_addr(y))
        return y

    # ---- convenience: operands outside the workspace ---------------------------------------------
    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        buf = self.view(x.dtype, x.numel())
        buf.copy_(x.reshape(-1))
        self.all_reduce_(buf)
        if out is None:
            out = torch.empty_like(x)
        out.reshape(-1).copy_(buf)
        return out

    def all_gather(self, shard: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        R = self.comm.world_size
        buf = self.view(shard.dtype, shard.numel() * R)
        self.all_gather_(shard, buf)
        if out is None:
            out = torch.empty((R,) + tuple(shard.shape), dtype=shard.dtype, device=shard.device)
        out.reshape(-1).copy_(buf)
        return out
