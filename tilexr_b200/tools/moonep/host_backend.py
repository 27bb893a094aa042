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

from typing import List

import torch

from ... import _C
from .contracts import MoonEPCase, RankInputs, StageArtifacts
from .planner_reference import dst_local_from_plans, reference_plan


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
        comm, rank = self.comm, self.comm.rank
        K, L, B, dt = case.top_k, case.local_experts, case.prefetch_slots, case.torch_dtype()
        if comm.world_size != case.ranks:
            raise ValueError(f"case {case.name} is written for {case.ranks} ranks")
        topk = self._all_gather(inputs.topk_experts_sk.to(torch.int32))
        plan = reference_plan(case, topk, rank)
        dst = plan["dst"].to(torch.int32).contiguous()
        dst_local = dst_local_from_plans(case, self._all_gather(dst), rank).to(torch.int32)
        plan["dst_local"] = dst_local

        rows32, w = _C.host_moon_dispatch(comm, inputs.hidden_sh.float().contiguous(), inputs.route_weights_sk.float().contiguous().reshape(-1),
                                          dst, dst_local, K)
        rows = rows32.to(dt)
        processed = rows if expert_fn is None else expert_fn(rows, plan)
        acc, wback = _C.host_moon_combine(comm, processed.float().contiguous(), w, dst, dst_local, case.tokens, K)

        prefetched = reduced = None
        if inputs.gate is not None:
            etc = plan["experts_to_copy"].to(torch.int64)
            gates = self._all_gather(inputs.gate.float())
            prefetched = torch.zeros((L + B,) + tuple(inputs.gate.shape[1:]), dtype=inputs.gate.dtype)
            prefetched[:L] = inputs.gate
            for b in range(B):
                e = int(etc[rank, b])
                if e >= 0:
                    prefetched[L + b] = gates[e // L][e % L].to(inputs.gate.dtype)
            grads = self._all_gather(inputs.grad_rows.float())
            reduced = inputs.grad_rows.clone().float()
            for src in range(case.ranks):
                for b in range(B):
                    e = int(etc[src, b])
                    if e >= 0 and e // L == rank and src != rank:
                        reduced[e % L] += grads[src][L + b]
            reduced[L:] = 0
        return StageArtifacts(plan=plan, dispatched_hidden=rows, dispatched_weights=w, prefetched_gate=prefetched,
                              combined_hidden=acc.to(dt), combined_weights=wback, reduced_grad=reduced)

    def close(self) -> None:
        pass
