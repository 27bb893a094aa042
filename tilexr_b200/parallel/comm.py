"""Communicator bring-up.

Four ways to get ranks, mirroring the init variants of the C API (csrc/include/tilexr_api.h;
reference: src/comm/comm_wrap.cpp:26-149):

* :func:`init_from_torch_distributed` -- one process per GPU, handles exchanged through the
  process group's ``Store`` (what ``torchrun`` users want);
* :func:`init_process` -- one process per GPU, handles exchanged through the library's own TCP
  bootstrap (``TILEXR_COMM_ID`` = ``ip:port`` of rank 0);
* :func:`init_emulated_world` -- several ranks on ONE GPU inside this process; every op on
  such a world must be issued for all ranks inside one :func:`group` block, which turns the
  per-rank calls into a single cooperative kernel.  Used by the single-GPU tests;
* :func:`init_host_memory` -- windows in POSIX shared memory and kernels on the CPU, for the
  no-GPU plumbing tests.
"""
from __future__ import annotations

import contextlib
from typing import Callable, List, Optional, Sequence

import torch

from .. import _C

Comm = _C.Comm

_store_calls = 0


def init_process(rank: int, world_size: int, comm_id: str = "", domain: int = 0, buffer_mb: int = 0,
                 device: int = -1) -> Comm:
    return _C.init_process(rank, world_size, comm_id, domain, buffer_mb, device)


def init_from_torch_distributed(group=None, buffer_mb: int = 0, domain: int = 0, device: Optional[int] = None,
                                host_memory: bool = False) -> Comm:
    """Creates this process's rank of a communicator that spans ``group`` (default: WORLD).

    ``host_memory=True`` gives the CPU plumbing communicator (works under the gloo backend).
    """
    import torch.distributed as dist

    global _store_calls
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialized")
    pg = group if group is not None else dist.group.WORLD
    rank = dist.get_rank(pg)
    world = dist.get_world_size(pg)
    store = dist.distributed_c10d._get_default_store()
    if device is None:
        device = torch.cuda.current_device() if (torch.cuda.is_available() and not host_memory) else -1
    ranks = dist.get_process_group_ranks(pg)
    prefix = f"tilexr/{domain}/{_store_calls}/{'-'.join(map(str, ranks))}"
    _store_calls += 1
    return _C.init_with_store(store, prefix, rank, world, domain, buffer_mb, device, host_memory)


def init_host_memory(rank: int, world_size: int, comm_id: str = "", domain: int = 0, buffer_mb: int = 64) -> Comm:
    return _C.init_host_memory(rank, world_size, comm_id, domain, buffer_mb)


@contextlib.contextmanager
def group():
    """Calls made inside are issued together when the block ends (needed for emulated worlds)."""
    _C.group_start()
    try:
        yield
    finally:
        _C.group_end()


class World:
    """All ranks of an emulated world, with helpers to run an op on every rank at once."""

    def __init__(self, comms: Sequence[Comm]):
        self.comms: List[Comm] = list(comms)

    @property
    def size(self) -> int:
        return len(self.comms)

    def __len__(self) -> int:
        return len(self.comms)

    def __getitem__(self, i: int) -> Comm:
        return self.comms[i]

    def run(self, fn: Callable[[Comm, int], object]) -> list:
        """``fn(comm, rank)`` for every rank inside one group; returns the per-rank results."""
        out = []
        with group():
            for r, c in enumerate(self.comms):
                out.append(fn(c, r))
        return out

    def symm_empty(self, shape, dtype) -> List[torch.Tensor]:
        return [c.symm_empty(list(shape), dtype) for c in self.comms]

    def check(self) -> None:
        """Raises if a bounded device wait of the last launches gave up on any rank."""
        torch.cuda.synchronize()
        for c in self.comms:
            status = c.device_status()
            if status != 0:
                c.print_dfx()
                raise RuntimeError(f"rank {c.rank}: device status {status} (see tilexr_comm_args.h TileXRDeviceStatus)")

    def destroy(self) -> None:
        for c in self.comms:
            c.destroy()


def init_emulated_world(world_size: int, device: int = 0, buffer_mb: int = 64) -> World:
    return World(_C.init_emulated(world_size, device, buffer_mb))
