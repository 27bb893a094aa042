"""Collectives over several NVSwitch domains: this library inside a node, `torch.distributed` between nodes.

A communicator of this library spans the GPUs that can load and store each other's memory (one NVLink / NVSwitch domain); ranks
on another host are refused at init.  The reference reaches other hosts through its RDMA transport (src/comm/udma); here the
second level is a process group of `torch.distributed` (NCCL over the NIC fabric), and every collective is cut into an
intra-node part on this library's kernels and an inter-node part that moves 1 / L of the bytes per rank (L = ranks per node):

    all_reduce       reduce-scatter in the node  ->  all-reduce of the shard across nodes (lane group)  ->  all-gather in the node
    all_gather       all-gather in the node      ->  all-gather of the node's block across nodes
    reduce_scatter   reduce-scatter in the node over the slices of every node  ->  reduce-scatter across nodes
    broadcast        across nodes on the root's lane  ->  in the node from that lane
    all_to_all       in the node by destination lane  ->  across nodes by destination node

Ranks are numbered node-major: global rank = node * L + local rank.  The "lane group" of a rank holds the ranks with its local
index on every node.  `ops` is the tensor-level collective module used inside the node (default: `tilexr_b200.ops.collectives`);
the CPU plumbing tests pass `HostMemoryOps`, which runs the same flows on host-memory communicators under gloo.
"""
from __future__ import annotations

from typing import List, Optional

import torch


class HostMemoryOps:
    """The intra-node collectives on a host-memory communicator (CPU tensors; sums in fp32), for the no-GPU plumbing mode.
    `tilexr_b200.ops.collectives` takes the same path for CPU tensors; this class only fixes the tile size."""

    def __init__(self, tile_bytes: int = 16384):
        self.tile_bytes = tile_bytes

    def all_reduce(self, comm, x):
        from ..ops import collectives

        return collectives.all_reduce(comm, x)

    def all_gather(self, comm, x):
        from .. import _C

        out = torch.empty((comm.world_size,) + tuple(x.shape), dtype=x.dtype)
        _C.host_all_gather(comm, x.contiguous(), out, self.tile_bytes)
        return out

    def reduce_scatter(self, comm, x):
        from ..ops import collectives

        return collectives.reduce_scatter(comm, x)

    def all_to_all(self, comm, x):
        from .. import _C

        return _C.host_all_to_all(comm, x.contiguous(), self.tile_bytes)

    def broadcast(self, comm, x, root=0):
        from .. import _C

        _C.host_broadcast(comm, x, root, self.tile_bytes)
        return x


class HierarchicalComm:
    """`intra_comm`: this library's communicator over the ranks of this node; `inter_group`: the `torch.distributed` group of this
    rank's lane (same local rank on every node), or None when there is one node."""

    def __init__(self, intra_comm, inter_group=None, ops=None, dist_module=None):
        if ops is None:
            from ..ops import collectives as ops
        if dist_module is None:
            import torch.distributed as dist_module
        self.intra, self.inter, self.ops, self.dist = intra_comm, inter_group, ops, dist_module
        self.local_rank, self.local_size = intra_comm.rank, intra_comm.world_size
        self.nodes = 1 if inter_group is None else dist_module.get_world_size(inter_group)
        self.node = 0 if inter_group is None else dist_module.get_rank(inter_group)
        self.rank = self.node * self.local_size + self.local_rank
        self.world_size = self.nodes * self.local_size

    # -- construction ----------------------------------------------------------------------------------------------
    @classmethod
    def from_torch_distributed(cls, local_world_size: Optional[int] = None, buffer_mb: int = 0, host_memory: bool = False, ops=None,
                               domain: int = 7) -> "HierarchicalComm":
        """Cuts the WORLD group into nodes of `local_world_size` consecutive ranks (default: LOCAL_WORLD_SIZE of the launcher's
        environment, else the whole world).  Every rank must call this: the groups are created collectively."""
        import os

        import torch.distributed as dist

        from .comm import init_from_torch_distributed

        world, rank = dist.get_world_size(), dist.get_rank()
        L = int(local_world_size or os.environ.get("LOCAL_WORLD_SIZE", world))
        if L <= 0 or world % L != 0:
            raise ValueError(f"{world} ranks do not divide into nodes of {L}")
        nodes = world // L
        node_groups = [dist.new_group(list(range(n * L, (n + 1) * L))) for n in range(nodes)]
        lane_groups = [dist.new_group([n * L + l for n in range(nodes)]) for l in range(L)] if nodes > 1 else [None] * L
        intra = init_from_torch_distributed(group=node_groups[rank // L], buffer_mb=buffer_mb, domain=domain, host_memory=host_memory)
        if ops is None and host_memory:
            ops = HostMemoryOps()
        return cls(intra, lane_groups[rank % L], ops)

    # -- collectives ------------------------------------------------------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over all ranks.  The element count must divide by the ranks per node."""
        if self.nodes == 1:
            return self.ops.all_reduce(self.intra, x)
        L = self.local_size
        flat = x.contiguous().reshape(-1)
        if flat.numel() % L != 0:
            raise ValueError("the element count must divide by the ranks of a node")
        shard = self.ops.reduce_scatter(self.intra, flat.view(L, -1)).reshape(-1)
        self.dist.all_reduce(shard, group=self.inter)
        return self.ops.all_gather(self.intra, shard).reshape(x.shape)

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """[world, *x.shape] in global rank order."""
        local = self.ops.all_gather(self.intra, x.contiguous())                      # [L, ...]
        if self.nodes == 1:
            return local
        blocks: List[torch.Tensor] = [torch.empty_like(local) for _ in range(self.nodes)]
        self.dist.all_gather(blocks, local.contiguous(), group=self.inter)
        return torch.cat(blocks, dim=0)

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """`x` holds world equal chunks along dim 0 (global rank order); returns the sum of chunk `rank` over all ranks."""
        if self.nodes == 1:
            return self.ops.reduce_scatter(self.intra, x)
        N, L = self.nodes, self.local_size
        if x.shape[0] % (N * L) != 0:
            raise ValueError("dim 0 must divide by the number of ranks")
        chunk = x.shape[0] // (N * L)
        rest = tuple(x.shape[1:])
        # [N, L, chunk, ...] -> lane-major [L, N, chunk, ...]: the node's ranks reduce, lane j keeps the slices of lane j on every node
        by_lane = x.contiguous().view((N, L, chunk) + rest).transpose(0, 1).contiguous()
        mine = self.ops.reduce_scatter(self.intra, by_lane.view((L * N * chunk,) + rest))      # [N * chunk, ...]: this node's partial sums
        parts = mine.view((N, chunk) + rest)
        if self.dist.get_backend(self.inter) == "gloo":
            # gloo has no reduce-scatter: all-reduce the node's partial sums and keep this node's slice (the CPU plumbing mode)
            total = parts.contiguous().clone()
            self.dist.all_reduce(total, group=self.inter)
            return total[self.node].contiguous()
        out = torch.empty_like(parts[0])
        self.dist.reduce_scatter(out, [p.contiguous() for p in parts.unbind(0)], group=self.inter)
        return out

    def broadcast(self, x: torch.Tensor, root: int = 0) -> torch.Tensor:
        if not 0 <= root < self.world_size:
            raise ValueError("root outside the communicator")
        root_lane = root % self.local_size
        if self.nodes > 1 and self.local_rank == root_lane:
            self.dist.broadcast(x, src=root, group=self.inter)           # the root is a member of this lane group
        return self.ops.broadcast(self.intra, x, root_lane)

    def all_to_all(self, x: torch.Tensor) -> torch.Tensor:
        """Equal split along dim 0: chunk g of `x` goes to global rank g; chunk s of the result came from global rank s."""
        if self.nodes == 1:
            return self.ops.all_to_all(self.intra, x)
        N, L = self.nodes, self.local_size
        if x.shape[0] % (N * L) != 0:
            raise ValueError("dim 0 must divide by the number of ranks")
        chunk = x.shape[0] // (N * L)
        rest = tuple(x.shape[1:])
        # hop 1, inside the node: everything addressed to lane j (on any node) goes to local rank j
        to_lane = x.contiguous().view((N, L, chunk) + rest).transpose(0, 1).contiguous()             # [L(dst lane), N(dst node), chunk]
        got = self.ops.all_to_all(self.intra, to_lane.view((L * N * chunk,) + rest))                   # [L(src lane), N(dst node), chunk]
        # hop 2, across nodes on this lane: the block addressed to node n goes to node n
        to_node = got.view((L, N, chunk) + rest).transpose(0, 1).contiguous()                          # [N(dst node), L(src lane), chunk]
        recv = torch.empty_like(to_node)
        self.dist.all_to_all_single(recv.view((N * L * chunk,) + rest), to_node.view((N * L * chunk,) + rest), group=self.inter)
        return recv.view((N * L * chunk,) + rest)                                                      # [N(src node), L(src lane), chunk] = global order

    def barrier(self) -> None:
        self.intra.barrier()
        if self.inter is not None:
            self.dist.barrier(group=self.inter)

    def destroy(self) -> None:
        self.intra.destroy()
