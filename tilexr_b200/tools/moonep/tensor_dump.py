"""Stage tensors on disk: dump what a backend produced for a case, compare two dumps offline (reference:
tools/moonep/tensor_dump.py).

A dump is a directory tree ``<root>/<case name>/rank<r>.pt`` (one ``torch.save`` dict per rank: the stage artifacts, the plan
tables under ``plan.<name>``, optionally the inputs under ``input.<name>``) with a ``manifest.json`` beside the rank files
that lists every tensor's shape, dtype and SHA-256.  Two runs (another build, another backend, another machine) are then
compared without either of them running: equal digests first, and for the tensors that differ the largest error and where the
first difference sits.

    python -m tilexr_b200.tools.moonep.tensor_dump show DIR
    python -m tilexr_b200.tools.moonep.tensor_dump compare DIR_A DIR_B [--rtol 0 --atol 0] [--ignore-missing]
"""
from __future__ import annotations

import argparse
import hashlib
import json
import pathlib
from typing import Dict, List, Optional

import torch

from .contracts import MoonEPCase, RankInputs, StageArtifacts

SCHEMA = "tilexr-moonep-dump-v1"


def _digest(t: torch.Tensor) -> str:
    c = t.detach().cpu().contiguous()
    return hashlib.sha256(c.view(torch.uint8).numpy().tobytes() if c.numel() else b"").hexdigest()


def flatten(artifacts: StageArtifacts, inputs: Optional[RankInputs] = None) -> Dict[str, torch.Tensor]:
    """One flat name -> CPU tensor mapping of a rank's artifacts (absent stages are left out)."""
    out: Dict[str, torch.Tensor] = {}
    for stage in StageArtifacts.STAGES:
        value = getattr(artifacts, stage)
        if stage == "plan":
            for k, v in value.items():
                if isinstance(v, torch.Tensor):
                    out[f"plan.{k}"] = v.detach().cpu()
        elif value is not None:
            out[stage] = value.detach().cpu()
    if inputs is not None:
        for k, v in vars(inputs).items():
            if isinstance(v, torch.Tensor):
                out[f"input.{k}"] = v.detach().cpu()
    return out


def dump_rank(root: str, case: MoonEPCase, rank: int, artifacts: StageArtifacts, inputs: Optional[RankInputs] = None,
              backend: str = "") -> pathlib.Path:
    """Writes rank ``rank``'s tensors of ``case`` and its part of the manifest; returns the rank file."""
    d = pathlib.Path(root) / case.name
    d.mkdir(parents=True, exist_ok=True)
    tensors = flatten(artifacts, inputs)
    path = d / f"rank{rank}.pt"
    torch.save(tensors, path)
    entry = {name: {"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", ""), "sha256": _digest(t)} for name, t in tensors.items()}
    (d / f"rank{rank}.manifest.json").write_text(json.dumps({"schema": SCHEMA, "case": case.name, "rank": rank, "backend": backend,
                                                             "shape": {"ranks": case.ranks, "tokens": case.tokens, "hidden": case.hidden,
                                                                       "top_k": case.top_k, "experts": case.experts,
                                                                       "prefetch_slots": case.prefetch_slots,
                                                                       "token_padding": case.token_padding, "dtype": case.dtype},
                                                             "tensors": entry}, indent=1))
    return path


def load_rank(root: str, case_name: str, rank: int) -> Dict[str, torch.Tensor]:
    return torch.load(pathlib.Path(root) / case_name / f"rank{rank}.pt", map_location="cpu")


def manifests(root: str) -> List[dict]:
    """Every rank manifest under ``root``, ordered by case and rank."""
    found = []
    for p in sorted(pathlib.Path(root).glob("*/rank*.manifest.json")):
        m = json.loads(p.read_text())
        if m.get("schema") != SCHEMA:
            raise ValueError(f"{p}: not a MoonEP tensor dump")
        found.append(m)
    return sorted(found, key=lambda m: (m["case"], m["rank"]))


def _compare_tensor(a: torch.Tensor, b: torch.Tensor, rtol: float, atol: float) -> dict:
    if a.shape != b.shape or a.dtype != b.dtype:
        return {"verdict": "layout", "a": f"{list(a.shape)} {a.dtype}", "b": f"{list(b.shape)} {b.dtype}"}
    if torch.equal(a, b):
        return {"verdict": "equal"}
    fa, fb = a.double().reshape(-1), b.double().reshape(-1)
    diff = (fa - fb).abs()
    bad = diff > (atol + rtol * fb.abs())
    bad |= torch.isnan(fa) != torch.isnan(fb)
    first = int(torch.nonzero(fa != fb)[0])
    row = {"max_abs": float(diff.nan_to_num(float("inf")).max()), "mismatched": int((fa != fb).sum()), "outside_tolerance": int(bad.sum()),
           "first_index": first, "a_at_first": float(fa[first]), "b_at_first": float(fb[first])}
    row["verdict"] = "close" if int(bad.sum()) == 0 else "differs"
    return row


def compare_dumps(root_a: str, root_b: str, rtol: float = 0.0, atol: float = 0.0) -> List[dict]:
    """One row per (case, rank, tensor) present in either dump.  Verdicts: equal (bit for bit, decided by the digests where
    both manifests have them), close (within tolerance), differs, layout (shape or dtype), missing (only in one dump)."""
    by_key_a = {(m["case"], m["rank"]): m for m in manifests(root_a)}
    by_key_b = {(m["case"], m["rank"]): m for m in manifests(root_b)}
    rows: List[dict] = []
    for key in sorted(set(by_key_a) | set(by_key_b)):
        case, rank = key
        ma, mb = by_key_a.get(key), by_key_b.get(key)
        if ma is None or mb is None:
            rows.append({"case": case, "rank": rank, "tensor": "*", "verdict": "missing", "only_in": "b" if ma is None else "a"})
            continue
        loaded_a = loaded_b = None
        for name in sorted(set(ma["tensors"]) | set(mb["tensors"])):
            ta, tb = ma["tensors"].get(name), mb["tensors"].get(name)
            row = {"case": case, "rank": rank, "tensor": name}
            if ta is None or tb is None:
                row.update(verdict="missing", only_in="b" if ta is None else "a")
            elif ta == tb:
                row.update(verdict="equal")
            else:
                if loaded_a is None:
                    loaded_a, loaded_b = load_rank(root_a, case, rank), load_rank(root_b, case, rank)
                row.update(_compare_tensor(loaded_a[name], loaded_b[name], rtol, atol))
            rows.append(row)
    return rows


def summarize(rows: List[dict], ignore_missing: bool = False) -> dict:
    """``ignore_missing``: tensors that only one dump has do not fail the comparison (a reference dump carries the inputs, a
    candidate's plan may carry tables of its own)."""
    counts: Dict[str, int] = {}
    for r in rows:
        counts[r["verdict"]] = counts.get(r["verdict"], 0) + 1
    accepted = ("equal", "close", "missing") if ignore_missing else ("equal", "close")
    return {"tensors": len(rows), "verdicts": counts, "ok": all(r["verdict"] in accepted for r in rows)}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = p.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("show")
    s.add_argument("root")
    c = sub.add_parser("compare")
    c.add_argument("a")
    c.add_argument("b")
    c.add_argument("--rtol", type=float, default=0.0)
    c.add_argument("--atol", type=float, default=0.0)
    c.add_argument("--all", action="store_true", help="also list the tensors that are equal")
    c.add_argument("--ignore-missing", action="store_true", help="tensors that only one dump has do not fail the comparison")
    args = p.parse_args(argv)
    if args.cmd == "show":
        for m in manifests(args.root):
            for name, t in m["tensors"].items():
                print(f"{m['case']} rank{m['rank']} {name}: {t['shape']} {t['dtype']} {t['sha256'][:12]}")
        return 0
    rows = compare_dumps(args.a, args.b, args.rtol, args.atol)
    for r in rows:
        if args.all or r["verdict"] not in (("equal", "missing") if args.ignore_missing else ("equal",)):
            print(json.dumps(r))
    summary = summarize(rows, args.ignore_missing)
    print(json.dumps(summary))
    return 0 if summary["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
