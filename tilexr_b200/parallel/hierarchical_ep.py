"""Expert parallelism over several NVSwitch domains: a hop between nodes on `torch.distributed`, then this library's
dispatch / combine inside the node.

A communicator of this library spans one NVLink / NVSwitch domain, so its expert-parallel kernels reach the experts of one
node.  With E experts over N nodes of L ranks (rank = node * L + lane, E / (N * L) experts per rank), a route to an expert of
another node crosses the NIC fabric exactly once in each direction, on the sender's lane:

    dispatch   1. routes are sorted by destination node; rows, node-local expert ids and the per-node counts go to the rank
                  with this rank's lane on each node (`all_to_all_single` on the lane group, uneven splits);
               2. what arrived is dispatched inside the node as top-1 routes over the node's E / N experts (the library's
                  kernel: rows land sorted by local expert, ready for a grouped GEMM).
    combine    2'. the expert outputs return inside the node to the rank that brought them in, unweighted;
               1'. they return across nodes on the lane, the source puts them back into route order and adds a token's K
                  rows, gate-weighted, in fp32 in route order.

The reference reaches other hosts through its RDMA transport inside the same kernels (src/comm/udma); here the second level is
a process group, which costs one host synchronisation per direction (the split sizes of the hop between nodes are host
integers) and is meant for the scale-out case, not for the NVLink fast path.  With one node, use `tilexr_b200.ops.ep` directly.

`ep_ops` is the adapter for the intra-node kernels: `DeviceEpOps` (CUDA tensors, `tilexr_b200.ops.ep`) or `HostEpOps` (fp32 CPU
tensors on a host-memory communicator, the no-GPU plumbing mode that the CPU tests run).
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional

import torch


@dataclasses.dataclass
class _IntraHandle:
    expand_x: torch.Tensor             # [max_recv_rows, H]; the first `recv_total` rows are valid, sorted by local expert
    expert_token_nums: torch.Tensor    # [experts per rank] rows per local expert
    recv_total: int
    state: object                      # what the adapter needs for the way back


class HostEpOps:
    """Intra-node dispatch / combine on a host-memory communicator (fp32 CPU tensors)."""

    def dispatch(self, comm, rows, ids, num_experts: int, max_recv_rows: int) -> _IntraHandle:
        from .. import _C

        expand, assist, nums, _counts, total = _C.host_ep_dispatch(comm, rows.contiguous(), ids.contiguous(), num_experts, max_recv_rows)
        return _IntraHandle(expand, nums, int(total), (assist, ids))

    def combine(self, comm, expert_out, h: _IntraHandle) -> torch.Tensor:
        from .. import _C

        assist, ids = h.state
        ones = torch.ones(ids.shape, dtype=torch.float32)
        return _C.host_ep_combine(comm, expert_out[: h.recv_total].contiguous(), assist, h.recv_total, ids, ones, int(h.expert_token_nums.numel()) * comm.world_size)


class DeviceEpOps:
    """Intra-node dispatch / combine on the device kernels (`tilexr_b200.ops.ep`), one route per row, no duplicates to fold."""

    def dispatch(self, comm, rows, ids, num_experts: int, max_recv_rows: int) -> _IntraHandle:
        from ..ops import ep

        d = ep.dispatch(comm, rows.contiguous(), num_experts=num_experts, top_k=1, expert_ids=ids.contiguous(), max_recv_rows=max_recv_rows, dedup=False)
        return _IntraHandle(d.expand_x, d.expert_token_nums, int(d.recv_total.item()), d)

    def combine(self, comm, expert_out, h: _IntraHandle) -> torch.Tensor:
        from ..ops import ep

        d = h.state
        ones = torch.ones((d.bs, 1), dtype=torch.float32, device=expert_out.device)
        return ep.combine(comm, expert_out, d, expert_scales=ones)


@dataclasses.dataclass
class HierarchicalDispatch:
    expand_x: torch.Tensor             # [max_recv_rows, H]; rows [0, recv_total) are this rank's, sorted by local expert
    expert_token_nums: torch.Tensor    # [E / (N * L)]
    recv_total: int
    # the way back
    intra: _IntraHandle
    order: torch.Tensor                # [bs * K] sorted position -> route index
    active: torch.Tensor               # [bs * K] bool, in sorted order
    send_splits: List[int]             # rows to each node (hop 1)
    recv_splits: List[int]             # rows from each node
    padded_rows: int                   # rows handed to the intra-node kernel (the same on every rank)
    bs: int
    top_k: int


class HierarchicalEP:
    """`hcomm`: a `HierarchicalComm` (its intra-node communicator and lane group are used)."""

    def __init__(self, hcomm, num_experts: int, ep_ops=None):
        W = hcomm.world_size
        if num_experts <= 0 or num_experts % W != 0:
            raise ValueError(f"{num_experts} experts do not divide over {W} ranks")
        self.h, self.E = hcomm, num_experts
        self.per_rank = num_experts // W
        self.per_node = self.per_rank * hcomm.local_size
        self.ops = ep_ops if ep_ops is not None else DeviceEpOps()

    # -- helpers ------------------------------------------------------------------------------------------------------
    def _lane_all_to_all(self, send: torch.Tensor, send_splits: List[int], recv_splits: List[int]) -> torch.Tensor:
        out = send.new_empty((sum(recv_splits),) + tuple(send.shape[1:]))
        if self.h.nodes == 1:
            out.copy_(send)
            return out
        self.h.dist.all_to_all_single(out, send.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits, group=self.h.inter)
        return out

    def _agree_max(self, value: int, device) -> int:
        """The largest `value` over all ranks of the job (the intra-node kernel's window layout depends on it)."""
        t = torch.tensor([value, 0, 0, 0], dtype=torch.int64, device=device)                  # 32 bytes: a whole vector for the gather
        if self.h.nodes > 1:
            self.h.dist.all_reduce(t, op=self.h.dist.ReduceOp.MAX, group=self.h.inter)
        return int(self.h.ops.all_gather(self.h.intra, t).max().item())

    # -- the two stages -----------------------------------------------------------------------------------------------
    def dispatch(self, x: torch.Tensor, expert_ids: torch.Tensor) -> HierarchicalDispatch:
        """`x` [bs, H]; `expert_ids` [bs, K] int32 global expert ids, negative = the route is inactive."""
        N = self.h.nodes
        bs, K = expert_ids.shape
        flat = expert_ids.reshape(-1).to(torch.int64)
        valid = (flat >= 0) & (flat < self.E)
        node = torch.where(valid, flat // self.per_node, torch.full_like(flat, N))            # inactive routes sort behind every node
        order = torch.argsort(node, stable=True)
        sorted_node = node[order]
        active = sorted_node < N
        send_splits = torch.bincount(sorted_node[active], minlength=N)[:N].tolist()
        sent = int(active.sum())
        rows = x[(order[:sent] // K)]
        local_ids = (flat[order[:sent]] - sorted_node[:sent] * self.per_node).to(torch.int32)

        counts = torch.tensor(send_splits, dtype=torch.int64, device=x.device)
        got = torch.empty_like(counts)
        if N > 1:
            self.h.dist.all_to_all_single(got, counts, group=self.h.inter)
        else:
            got.copy_(counts)
        recv_splits = got.tolist()                                                              # host integers: one synchronisation
        rows_in = self._lane_all_to_all(rows, send_splits, recv_splits)
        ids_in = self._lane_all_to_all(local_ids, send_splits, recv_splits)

        M = int(rows_in.shape[0])
        padded = max(1, self._agree_max(M, x.device))
        if M < padded:                                                                          # the kernel takes the same row count on every rank
            rows_in = torch.cat([rows_in, rows_in.new_zeros((padded - M,) + tuple(rows_in.shape[1:]))])
            ids_in = torch.cat([ids_in, ids_in.new_full((padded - M,), -1)])
        intra = self.ops.dispatch(self.h.intra, rows_in, ids_in.view(-1, 1), self.per_node, padded * self.h.local_size)
        return HierarchicalDispatch(intra.expand_x, intra.expert_token_nums, intra.recv_total, intra, order, active, send_splits, recv_splits,
                                    padded, bs, K)

    def combine(self, expert_out: torch.Tensor, d: HierarchicalDispatch, expert_scales: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`expert_out`: one output row per row of `d.expand_x` (the first `d.recv_total` count).  `expert_scales` [bs, K] fp32
        gate weights (default: ones).  Returns [bs, H] in the type of `expert_out`."""
        back = self.ops.combine(self.h.intra, expert_out, d.intra)                              # [padded, H], in the order the rows came in
        back = back[: sum(d.recv_splits)]
        home = self._lane_all_to_all(back, d.recv_splits, d.send_splits)                        # sorted-route order at the source
        n = d.bs * d.top_k
        sent = home.shape[0]
        per_route = torch.zeros((n,) + tuple(home.shape[1:]), dtype=torch.float32, device=home.device)
        per_route[d.order[:sent]] = home.float()
        w = torch.ones(d.bs, d.top_k, dtype=torch.float32, device=home.device) if expert_scales is None else expert_scales.float()
        y = torch.zeros((d.bs,) + tuple(home.shape[1:]), dtype=torch.float32, device=home.device)
        per_route = per_route.view((d.bs, d.top_k) + tuple(home.shape[1:]))
        for k in range(d.top_k):                                                                # route order: the order the sum is defined in
            y += w[:, k].reshape((-1,) + (1,) * (y.dim() - 1)) * per_route[:, k]
        return y.to(expert_out.dtype)
