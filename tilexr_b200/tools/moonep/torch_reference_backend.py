"""Pure-torch reference of the five MoonEP stages (reference: tools/moonep/torch_npu_backend.py and the CPU
stage reference tests/moonep/reference/moonep_stage_reference.cpp:86-475).

Every rank gathers all ranks' inputs with `torch.distributed` (gloo with CPU tensors, or NCCL), then computes
its own expected outputs; no stage of the library under test is involved.  Semantics:

* dispatch: route i of source s with `dst[i] = r * NvS + slot` puts `hidden[s][i // K]` and `weights[s][i]` into
  row `slot` of rank r; rows nobody fills are zero.
* prefetch: slot b of rank r with `experts_to_copy[r, b] = e >= 0` receives the rows of expert e from its owner.
* combine: the inverse of dispatch, K rows per token summed in fp32 in route order and rounded once; weights
  return bit-exact.
* reduce-grad: the owner of expert e adds, in ascending (source rank, slot), the slot rows of every rank that
  borrowed e; all slot rows are cleared afterwards.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .contracts import MoonEPCase, RankInputs, StageArtifacts
from .planner_reference import dst_local_from_plans, reference_plan


def _gather(t: Optional[torch.Tensor], group) -> List[Optional[torch.Tensor]]:
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return [None if t is None else t.cpu()]
    out: List[Optional[torch.Tensor]] = [None] * world
    dist.all_gather_object(out, None if t is None else t.cpu(), group=group)
    return out


class TorchReferenceBackend:
    name = "torch-reference"

    def __init__(self, group=None, identity_expert: bool = True):
        self.group = group
        self.identity_expert = identity_expert

    def run(self, case: MoonEPCase, inputs: RankInputs, expert_rows=None) -> StageArtifacts:
        rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        R, K, n, nvs, L, B = case.ranks, case.top_k, case.routes, case.nvs, case.local_experts, case.prefetch_slots
        topk = _gather(inputs.topk_experts_sk, self.group)
        hidden = _gather(inputs.hidden_sh, self.group)
        weights = _gather(inputs.route_weights_sk, self.group)
        plans = [reference_plan(case, topk, r) for r in range(R)]
        plan = plans[rank]
        dsts = [p["dst"] for p in plans]
        plan["dst_local"] = dst_local_from_plans(case, dsts, rank).to(torch.int32)      # the dtype of the planner kernel's table

        # dispatch, for every rank (combine needs what the others hold)
        rows = [torch.zeros(nvs, case.hidden, dtype=case.torch_dtype()) for _ in range(R)]
        wrow = [torch.zeros(nvs, dtype=torch.float32) for _ in range(R)]
        for src in range(R):
            raw = dsts[src].to(torch.int64)
            keep = raw >= 0
            r_of, slot = raw[keep] // nvs, raw[keep] % nvs
            route = torch.nonzero(keep).reshape(-1)
            for r in range(R):
                m = r_of == r
                rows[r][slot[m]] = hidden[src][route[m] // K]
                wrow[r][slot[m]] = weights[src].reshape(-1)[route[m]]
        processed = rows if expert_rows is None else expert_rows

        # combine for this rank
        raw = dsts[rank].to(torch.int64)
        acc = torch.zeros(case.tokens, case.hidden, dtype=torch.float32)
        wback = torch.zeros(n, dtype=torch.float32)
        for i in range(n):                      # route order: the order the fp32 sum is defined in
            v = int(raw[i])
            if v < 0:
                continue
            r, slot = divmod(v, nvs)
            acc[i // K] += processed[r][slot].float()
            wback[i] = wrow[r][slot]
        combined = acc.to(case.torch_dtype())

        prefetched = reduced = None
        if inputs.gate is not None:
            gates = _gather(inputs.gate, self.group)
            etc = plan["experts_to_copy"].to(torch.int64)
            prefetched = torch.zeros((L + B,) + tuple(inputs.gate.shape[1:]), dtype=inputs.gate.dtype)
            prefetched[:L] = gates[rank]
            for b in range(B):
                e = int(etc[rank, b])
                if e >= 0:
                    prefetched[L + b] = gates[e // L][e % L]
            grads = _gather(inputs.grad_rows, self.group)
            reduced = grads[rank].clone().float()
            for src in range(R):
                for b in range(B):
                    e = int(etc[src, b])
                    if e >= 0 and e // L == rank and src != rank:
                        reduced[e % L] += grads[src][L + b].float()
            reduced[L:] = 0
        return StageArtifacts(plan=plan, dispatched_hidden=rows[rank], dispatched_weights=wrow[rank],
                              prefetched_gate=prefetched, combined_hidden=combined,
                              combined_weights=wback.view(case.tokens, K), reduced_grad=reduced)

    def close(self) -> None:
        pass
