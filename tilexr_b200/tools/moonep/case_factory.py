"""Deterministic inputs for a case (reference: tools/moonep/case_factory.py) and the case files."""
from __future__ import annotations

import json
import pathlib
from typing import Dict, List

import torch

from .contracts import MoonEPCase, RankInputs

CASE_DIR = pathlib.Path(__file__).resolve().parent / "cases"


def load_cases(name_or_path: str) -> List[MoonEPCase]:
    path = pathlib.Path(name_or_path)
    if not path.exists():
        path = CASE_DIR / f"{name_or_path}.json"
    cases = [MoonEPCase(**c) for c in json.loads(path.read_text())["cases"]]
    for c in cases:
        c.validate()
    return cases


def routing(case: MoonEPCase, rank: int) -> torch.Tensor:
    """[S, K] int32 expert ids; the first E/8 experts are `skew` times as likely (a hot-expert workload)."""
    g = torch.Generator().manual_seed(case.seed * 1000003 + rank)
    p = torch.ones(case.experts)
    p[: max(1, case.experts // 8)] = case.skew
    return torch.multinomial(p, case.routes, replacement=True, generator=g).to(torch.int32).view(case.tokens, case.top_k)


def make_inputs(case: MoonEPCase, rank: int, device: str = "cpu") -> RankInputs:
    g = torch.Generator().manual_seed(case.seed * 7919 + 17 * rank + 1)
    dt = case.torch_dtype()
    hidden = torch.randn(case.tokens, case.hidden, generator=g).to(dt)
    weights = torch.rand(case.tokens, case.top_k, generator=g)
    inputs = RankInputs(hidden.to(device), weights.to(device), routing(case, rank).to(device))
    if case.ffn > 0:
        L, B = case.local_experts, case.prefetch_slots
        mk = lambda: (torch.randn(L, case.ffn, case.hidden, generator=g) * 0.05).to(dt).to(device)
        inputs.gate, inputs.up, inputs.down = mk(), mk(), mk()
        inputs.grad_rows = torch.randn(L + B, case.ffn, case.hidden, generator=g).to(device)
    return inputs


def snapshot(inputs: RankInputs) -> Dict[str, torch.Tensor]:
    return {k: v.clone() for k, v in vars(inputs).items() if isinstance(v, torch.Tensor)}


def unchanged(inputs: RankInputs, snap: Dict[str, torch.Tensor]) -> List[str]:
    """Names of inputs that a backend modified."""
    return [k for k, v in snap.items() if not torch.equal(getattr(inputs, k), v)]
