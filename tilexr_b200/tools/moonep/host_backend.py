"""The five MoonEP stages on a host-memory communicator: the harness without a GPU.

The rows travel through the same windows, flags, launch epochs and reuse guard as on the device (the host build of the
flag primitives); only the copies are `memcpy`.  What each stage uses:

* planning: every rank's routing is exchanged with the host all-gather, then the library's host build of the planner
  produces this rank's plan; the plans' destinations are exchanged the same way for the inverse table.
* dispatch / combine: `host_moon_dispatch` / `host_moon_combine` (rows placed by the plan behind one flag per source; rows
  returned to the route's position behind one flag per route, a token's K rows added in route order in fp32, rounded once).
* prefetch / reduce-grad: the owners' expert rows, or every rank's gradient rows, are exchanged with the host all-gather;
  the slots are filled, or the owner adds the borrowers' rows in ascending (source rank, slot).

16-bit inputs are widened to fp32 for the transport (exact) and narrowed at the end.
"""
from __future__ import annotations

import types
from typing import List, Optional

import torch

from ... import _C
from .contracts import MoonEPCase, RankInputs, StageArtifacts
from .planner_reference import dst_local_from_plans, reference_plan


class HostPlan(types.SimpleNamespace):
    """dst, dst_local (int32), experts_to_copy [R, B], remote_stats, tables: the planner's full dictionary."""


class HostStageBuffer:
    """The stage methods of `TileXRMoonEPBuffer` (planning, dispatch, prefetch_weight, combine, reduce_grad) on a host-memory
    communicator, blocking, for drivers that only need those methods (the correctness backend below, the model flow)."""

    def __init__(self, comm, case: MoonEPCase, tile_bytes: int = 16384):
        if comm.physical_info()["link"] != "host_memory":
            raise ValueError("the host stages need a communicator made with host_memory=True")
        if comm.world_size != case.ranks:
            raise ValueError(f"case {case.name} is written for {case.ranks} ranks")
        self.comm, self.case, self.tile_bytes = comm, case, tile_bytes
        self.weights_nvs: Optional[torch.Tensor] = None          # route weights as the last dispatch delivered them

    def all_gather(self, t: torch.Tensor) -> List[torch.Tensor]:
        """Every rank's `t` (equal shapes), through the window."""
        flat = t.contiguous().reshape(-1)
        out = torch.empty((self.comm.world_size,) + tuple(flat.shape), dtype=flat.dtype)
        _C.host_all_gather(self.comm, flat, out, self.tile_bytes)
        return [out[r].view(t.shape) for r in range(self.comm.world_size)]

    def planning(self, topk_experts_sk: torch.Tensor) -> HostPlan:
        case, rank = self.case, self.comm.rank
        tables = reference_plan(case, self.all_gather(topk_experts_sk.to(torch.int32)), rank)
        dst = tables["dst"].to(torch.int32).contiguous()
        dst_local = dst_local_from_plans(case, self.all_gather(dst), rank).to(torch.int32)
        tables["dst_local"] = dst_local
        return HostPlan(dst=dst, dst_local=dst_local, experts_to_copy=tables["experts_to_copy"], remote_stats=tables.get("remote_stats"), tables=tables)

    def dispatch(self, hidden: torch.Tensor, route_weights: Optional[torch.Tensor], plan: HostPlan):
        w = None if route_weights is None else route_weights.float().contiguous().reshape(-1)
        rows, wn = _C.host_moon_dispatch(self.comm, hidden.float().contiguous(), w, plan.dst, plan.dst_local, self.case.top_k)
        if wn is not None:
            self.weights_nvs = wn
        return rows.to(hidden.dtype), wn

    def combine(self, plan: HostPlan, rows: torch.Tensor, weights_nvs: Optional[torch.Tensor] = None):
        acc, wback = _C.host_moon_combine(self.comm, rows.float().contiguous(), weights_nvs, plan.dst, plan.dst_local, self.case.tokens, self.case.top_k)
        return acc.to(rows.dtype), wback

    def prefetch_weight(self, plan: HostPlan, projections) -> None:
        """Slot L + b of every projection tensor ([L + B, ...], own experts in front) receives the rows of expert
        experts_to_copy[rank, b] from its owner; slots nobody fills are zeroed."""
        L, B, rank = self.case.local_experts, self.case.prefetch_slots, self.comm.rank
        etc = plan.experts_to_copy.to(torch.int64)
        for t in (projections.gate, projections.up, projections.down):
            if t is None:
                continue
            owners = self.all_gather(t[:L].float())
            for b in range(B):
                e = int(etc[rank, b])
                if e >= 0:
                    t[L + b] = owners[e // L][e % L].to(t.dtype)
                else:
                    t[L + b] = 0

    def reduce_grad(self, plan: HostPlan, grads) -> None:
        """The owner of expert e adds, in ascending (source rank, slot), the slot rows of every rank that borrowed e; all slot
        rows are cleared afterwards (fp32 gradient tensors [L + B, ...])."""
        L, B, rank = self.case.local_experts, self.case.prefetch_slots, self.comm.rank
        etc = plan.experts_to_copy.to(torch.int64)
        for t in (grads.gate, grads.up, grads.down):
            if t is None:
                continue
            every = self.all_gather(t.float())
            for src in range(self.case.ranks):
                for b in range(B):
                    e = int(etc[src, b])
                    if e >= 0 and e // L == rank and src != rank:
                        t[e % L] += every[src][L + b]
            t[L:] = 0

    def synchronize(self) -> None:
        pass

    def close(self) -> None:
        pass


class HostMemoryBackend:
    name = "tilexr-host-memory"

    def __init__(self, comm, tile_bytes: int = 16384):
        if comm.physical_info()["link"] != "host_memory":
            raise ValueError("HostMemoryBackend needs a communicator made with host_memory=True")
        self.comm, self.tile_bytes = comm, tile_bytes

    def _all_gather(self, t: torch.Tensor) -> List[torch.Tensor]:
        """Every rank's `t` (equal shapes), through the window."""
        flat = t.contiguous().reshape(-1)
        out = torch.empty((self.comm.world_size,) + tuple(flat.shape), dtype=flat.dtype)
        _C.host_all_gather(self.comm, flat, out, self.tile_bytes)
        return [out[r].view(t.shape) for r in range(self.comm.world_size)]

    def run(self, case: MoonEPCase, inputs: RankInputs, expert_fn=None) -> StageArtifacts:
        buf = HostStageBuffer(self.comm, case, self.tile_bytes)
        L, B = case.local_experts, case.prefetch_slots
        plan = buf.planning(inputs.topk_experts_sk)
        rows, w = buf.dispatch(inputs.hidden_sh, inputs.route_weights_sk, plan)
        processed = rows if expert_fn is None else expert_fn(rows, plan.tables)
        combined, wback = buf.combine(plan, processed, w)
        prefetched = reduced = None
        if inputs.gate is not None:
            prefetched = torch.zeros((L + B,) + tuple(inputs.gate.shape[1:]), dtype=inputs.gate.dtype)
            prefetched[:L] = inputs.gate
            buf.prefetch_weight(plan, types.SimpleNamespace(gate=prefetched, up=None, down=None))
            reduced = inputs.grad_rows.clone().float()
            buf.reduce_grad(plan, types.SimpleNamespace(gate=reduced, up=None, down=None))
        return StageArtifacts(plan=plan.tables, dispatched_hidden=rows, dispatched_weights=w, prefetched_gate=prefetched,
                              combined_hidden=combined, combined_weights=wback, reduced_grad=reduced)

    def close(self) -> None:
        pass
