"""CPU planner reference and plan invariants (reference: tools/moonep/planner_reference.py:104-310,
tests/moonep_planner/reference/planner_reference.cpp:63-279).  The algorithm itself is the library's host
build of the shared planner header; this module adds the checks every plan must pass."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ... import _C
from .contracts import MoonEPCase


def reference_plan(case: MoonEPCase, all_topk: Sequence[torch.Tensor], rank: int) -> Dict[str, torch.Tensor]:
    """Plan of `rank` given every rank's [S, K] routing."""
    stacked = torch.stack([t.reshape(-1).to(torch.int32).cpu() for t in all_topk]).contiguous()
    return dict(_C.moonep_reference_plan(stacked, rank, case.tokens, case.top_k, case.experts, case.prefetch_slots,
                                         case.token_padding))


def reference_plan_v2(case: MoonEPCase, all_topk: Sequence[torch.Tensor], rank: int, global_rank_ids: Optional[Sequence[int]] = None,
                      nvs: Optional[int] = None, route_limit_per_pair: int = 0) -> Dict[str, torch.Tensor]:
    """Plan of `rank` from the topology-aware planner's CPU oracle (the library's host build of the V2 algorithm source),
    in the key names the invariants below use.  ``dst`` keeps the duplicate encoding (~raw); ``code`` is the plan status."""
    R, E = case.ranks, case.experts
    topk = [t.reshape(case.tokens, case.top_k).to(torch.int32).cpu().contiguous() for t in all_topk]
    tpe = torch.stack([torch.bincount(t.reshape(-1).to(torch.int64), minlength=E) for t in topk]).to(torch.int32).contiguous()
    gids = torch.tensor(list(global_rank_ids) if global_rank_ids is not None else list(range(R)), dtype=torch.int32)
    if nvs is None:
        nvs = case.routes + (E + case.prefetch_slots) * (case.token_padding - 1)
    d = dict(_C.moonep_plan_v2_reference(rank, topk[rank], tpe, gids, case.prefetch_slots, nvs, case.token_padding, route_limit_per_pair))
    d["slots_of_this_rank"] = d["experts_to_copy"]
    d["experts_to_copy"] = d["remote_experts"]          # [R, B]: every rank's slots, as the V3 plan reports them
    d["NvS"] = nvs
    return d


def dst_local_from_plans(case: MoonEPCase, dsts: Sequence[torch.Tensor], rank: int) -> torch.Tensor:
    """Inverse map of `rank`: slot -> src * N + route, -1 for padding."""
    nvs, n = case.nvs, case.routes
    out = torch.full((nvs,), -1, dtype=torch.int64)
    for src, dst in enumerate(dsts):
        raw = dst.to(torch.int64).cpu()
        here = (raw >= 0) & (raw // nvs == rank)
        idx = torch.nonzero(here).reshape(-1)
        out[raw[idx] % nvs] = src * n + idx
    return out


def check_plan_invariants(case: MoonEPCase, plans: Sequence[Dict[str, torch.Tensor]]) -> List[str]:
    """Violations over the plans of all ranks (empty list = fine)."""
    bad: List[str] = []
    nvs, n, L, B = int(plans[0].get("NvS", case.nvs)), case.routes, case.local_experts, case.prefetch_slots
    seen = [set() for _ in range(case.ranks)]
    for src, p in enumerate(plans):
        dst = p["dst"].to(torch.int64).cpu()
        if dst.numel() != n:
            bad.append(f"rank {src}: dst has {dst.numel()} entries, want {n}")
            continue
        for i, raw in enumerate(dst.tolist()):
            if raw < 0:
                raw = ~raw                      # duplicate of an earlier route of the token to that rank
            r, slot = divmod(raw, nvs)
            if not 0 <= r < case.ranks:
                bad.append(f"rank {src} route {i}: destination rank {r}")
            elif dst[i] >= 0:
                if slot in seen[r]:
                    bad.append(f"rank {src} route {i}: slot {slot} of rank {r} used twice")
                seen[r].add(slot)
    for r, p in enumerate(plans):
        cu = p["cu_seqlens"].to(torch.int64).cpu()
        if (cu[1:] < cu[:-1]).any():
            bad.append(f"rank {r}: cu_seqlens not monotone")
        if len(seen[r]) > nvs:
            bad.append(f"rank {r}: receives {len(seen[r])} rows, capacity {nvs}")
        etc = p["experts_to_copy"].to(torch.int64).cpu()
        if tuple(etc.shape) != (case.ranks, B):
            bad.append(f"rank {r}: experts_to_copy shape {tuple(etc.shape)}")
        for b, ex in enumerate(etc[r].tolist()):
            if ex >= 0 and ex // L == r:
                bad.append(f"rank {r}: slot {b} prefetches its own expert {ex}")
    ref = plans[0]["experts_to_copy"].cpu()
    for r, p in enumerate(plans[1:], 1):
        if not torch.equal(p["experts_to_copy"].cpu(), ref):
            bad.append(f"rank {r}: experts_to_copy differs from rank 0 (every rank must see the same table)")
    return bad
