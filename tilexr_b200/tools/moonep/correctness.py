"""Reference-vs-candidate comparison of the stage artifacts (reference: tools/moonep/correctness.py,
`CorrectnessRunner`): exact, close and ULP comparisons per artifact, input immutability, and rank-wide
agreement on the verdict."""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .case_factory import make_inputs, snapshot, unchanged
from .contracts import MoonEPBackend, MoonEPCase, StageArtifacts

# How each artifact is compared: plan tensors and weights are bit-exact; rows that are pure copies are exact;
# the combined hidden is a sum of K bf16 rows in fp32 rounded once, so one ULP of the output type is allowed
# for backends that add in another (documented) order; the gradient sum is fp32 in a fixed order: exact.
POLICY = {
    "plan": "exact",
    "dispatched_hidden": "exact",
    "dispatched_weights": "exact",
    "prefetched_gate": "exact",
    "combined_hidden": "ulp:1",
    "combined_weights": "exact",
    "reduced_grad": "exact",
}
PLAN_KEYS = ("dst", "cu_seqlens", "experts_to_copy", "zero_fill_ranges", "remote_stats")


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance in units in the last place between two tensors of one 16-bit float type."""
    if a.numel() == 0:
        return 0
    ia = a.contiguous().view(torch.int16).to(torch.int32)
    ib = b.contiguous().view(torch.int16).to(torch.int32)
    ia = torch.where(ia < 0, -(ia & 0x7fff), ia)          # sign-magnitude -> ordered integers
    ib = torch.where(ib < 0, -(ib & 0x7fff), ib)
    return int((ia - ib).abs().max())


@dataclasses.dataclass
class StageVerdict:
    stage: str
    ok: bool
    detail: str = ""


def compare(stage: str, want, got) -> StageVerdict:
    if want is None and got is None:
        return StageVerdict(stage, True, "not part of this case")
    if (want is None) != (got is None):
        return StageVerdict(stage, False, "one side is missing")
    if stage == "plan":
        for k in PLAN_KEYS:
            if k in want and k in got and not torch.equal(want[k].cpu().to(torch.int64), got[k].cpu().to(torch.int64)):
                return StageVerdict(stage, False, f"plan tensor {k} differs")
        return StageVerdict(stage, True)
    want, got = want.cpu(), got.cpu()
    if want.shape != got.shape or want.dtype != got.dtype:
        return StageVerdict(stage, False, f"shape/dtype {tuple(got.shape)} {got.dtype}, want {tuple(want.shape)} {want.dtype}")
    policy = POLICY[stage]
    if policy == "exact":
        if torch.equal(want, got):
            return StageVerdict(stage, True)
        bad = int((want != got).sum())
        return StageVerdict(stage, False, f"{bad} elements differ (bit-exact comparison)")
    limit = int(policy.split(":")[1])
    if want.element_size() == 2:
        d = ulp_distance(want, got)
        return StageVerdict(stage, d <= limit, f"max distance {d} ulp (limit {limit})")
    ok = torch.allclose(want, got, rtol=1e-6, atol=1e-6)
    return StageVerdict(stage, ok, "fp32 close comparison")


class CorrectnessRunner:
    def __init__(self, reference: MoonEPBackend, candidate: MoonEPBackend, group=None, device: str = "cpu", dump_dir: str = ""):
        """``dump_dir``: both sides' artifacts of every case go to ``<dump_dir>/reference`` and ``<dump_dir>/candidate``
        (tensor_dump.py), for an offline look at a failure or a comparison with another build's run."""
        self.reference, self.candidate, self.group, self.device = reference, candidate, group, device
        self.dump_dir = dump_dir

    def run_case(self, case: MoonEPCase) -> Dict[str, object]:
        rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        inputs = make_inputs(case, rank, self.device)
        snap = snapshot(inputs)
        want: StageArtifacts = self.reference.run(case, inputs)
        touched = unchanged(inputs, snap)
        got: StageArtifacts = self.candidate.run(case, inputs)
        touched += [f"{k} (candidate)" for k in unchanged(inputs, snap)]
        if self.dump_dir:
            from . import tensor_dump

            tensor_dump.dump_rank(f"{self.dump_dir}/reference", case, rank, want, inputs, getattr(self.reference, "name", "reference"))
            tensor_dump.dump_rank(f"{self.dump_dir}/candidate", case, rank, got, None, getattr(self.candidate, "name", "candidate"))
        verdicts: List[StageVerdict] = [compare(s, getattr(want, s), getattr(got, s)) for s in StageArtifacts.STAGES]
        if touched:
            verdicts.append(StageVerdict("inputs_immutable", False, "modified: " + ", ".join(touched)))
        else:
            verdicts.append(StageVerdict("inputs_immutable", True))
        ok_here = all(v.ok for v in verdicts)
        ok_all = self._agree(ok_here)
        return {"case": case.name, "rank": rank, "ok": ok_here, "ok_all_ranks": ok_all,
                "stages": [dataclasses.asdict(v) for v in verdicts]}

    def _agree(self, ok: bool) -> bool:
        """Every rank learns whether every rank passed (a case passes only as a whole)."""
        if not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return ok
        flags: List[Optional[bool]] = [None] * dist.get_world_size(self.group)
        dist.all_gather_object(flags, ok, group=self.group)
        return all(flags)
