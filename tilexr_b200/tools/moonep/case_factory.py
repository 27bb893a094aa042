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


def select_cases(cases: List[MoonEPCase], case_ids: str = "") -> List[MoonEPCase]:
    """``case_ids``: comma-separated case names or 1-based positions in the file, in the order wanted; empty keeps all
    (reference: tools/moonep/config.py:118-138)."""
    if not case_ids:
        return list(cases)
    by_name = {c.name: c for c in cases}
    if len(by_name) != len(cases):
        raise ValueError("case names must be unique")
    picked = []
    for item in (x.strip() for x in case_ids.split(",")):
        if not item:
            continue
        if item.isdigit():
            n = int(item)
            if not 1 <= n <= len(cases):
                raise ValueError(f"case number must be in [1, {len(cases)}]: {item}")
            picked.append(cases[n - 1])
        elif item in by_name:
            picked.append(by_name[item])
        else:
            raise ValueError(f"unknown case: {item}")
    return picked


OVERRIDABLE = ("tokens", "hidden", "top_k", "experts", "prefetch_slots", "token_padding", "ffn", "skew", "seed", "dtype")


def apply_overrides(case: MoonEPCase, overrides: Dict[str, object]) -> MoonEPCase:
    """The case with the given fields replaced (None values are ignored) and validated again; the name says what changed."""
    import dataclasses

    changes = {k: v for k, v in overrides.items() if v is not None}
    unknown = [k for k in changes if k not in OVERRIDABLE]
    if unknown:
        raise ValueError(f"not a case field that can be overridden: {', '.join(unknown)}")
    if not changes:
        return case
    tag = ",".join(f"{k}={changes[k]}" for k in sorted(changes))
    out = dataclasses.replace(case, name=f"{case.name}[{tag}]", **changes)
    out.validate()
    return out


def add_case_arguments(parser) -> None:
    """``--case-ids`` and one flag per overridable field, for the harness entry points."""
    parser.add_argument("--case-ids", default="", help="comma-separated case names or 1-based numbers (default: every case of the file)")
    for name, kind in (("tokens", int), ("hidden", int), ("top-k", int), ("experts", int), ("prefetch-slots", int), ("token-padding", int),
                       ("ffn", int), ("skew", float), ("seed", int), ("dtype", str)):
        parser.add_argument(f"--{name}", type=kind, default=None, help=f"override the cases' {name.replace('-', '_')}")


def overrides_from_args(args) -> Dict[str, object]:
    return {k: getattr(args, k, None) for k in OVERRIDABLE}


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
